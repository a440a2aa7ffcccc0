// build: precise-math
// Image filter kernels on RGBA fp32 images [H, W, 4] (values nominally in [0, 1]); one thread per pixel, 16 x 16 blocks,
// edge-clamped loads. Compute only: no graphics API is involved anywhere. This file is compiled WITHOUT fast-math and
// WITHOUT multiply-add contraction: several filters hash coordinates through fract() of large products, where one
// differently rounded bit changes the result completely, so every operation rounds like the fp32 CPU statement of the
// same formula does.
//
// Filters: SmartDenoise, HQDN3D (single frame), Guided (self-guided, 5 passes), Deband, ColorBalance, CAS,
// USM (separable gaussian), LUT3D (trilinear), WaterRipple, Soul, Sway, Star, Lighting, Jitter.
// Formulas: shader_denoise_ref.py:63-300, shader_color_adv_ref.py:55-215, shader_effects_ref.py:70-400
// (CUDA-style originals shader_denoise.mojo:90-371, shader_color_adv.mojo:93-270, shader_effects.mojo:109-598).
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "kernels_api.h"

namespace mdb {
namespace filt {

struct Img {
  const float* p;
  int H, W;
  __device__ __forceinline__ float ld(int x, int y, int ch) const {
    x = min(max(x, 0), W - 1);
    y = min(max(y, 0), H - 1);
    return p[(static_cast<long long>(y) * W + x) * 4 + ch];
  }
};
__device__ __forceinline__ float clamp01(float v) { return fminf(fmaxf(v, 0.f), 1.f); }
__device__ __forceinline__ float gfloor(float x) { return floorf(x); }
__device__ __forceinline__ float gfract(float x) { return x - floorf(x); }
__device__ __forceinline__ float gmod(float x, float y) { return x - y * floorf(x / y); }
__device__ __forceinline__ float smoothstep(float e0, float e1, float x) {
  float t = clamp01((x - e0) / (e1 - e0));
  return t * t * (3.f - 2.f * t);
}
#define PIXEL_XY()                                         \
  const int x = blockIdx.x * blockDim.x + threadIdx.x;     \
  const int y = blockIdx.y * blockDim.y + threadIdx.y;     \
  if (x >= in.W || y >= in.H) return;                      \
  float* o = out + (static_cast<long long>(y) * in.W + x) * 4;

// ---- denoise group ----------------------------------------------------------------------------------------------------
__global__ void smartdenoise_kernel(Img in, float* out, float sigma, float ksigma, float threshold) {
  PIXEL_XY();
  const float inv_gamma = 0.454545454545455f;
  const float radius = rintf(ksigma * sigma);
  const float radQ = radius * radius;
  const float invSigmaQx2 = 0.5f / (sigma * sigma);
  const float invSigmaQx2PI = 0.31830988618379067f * invSigmaQx2;
  const float invThresholdSqx2 = 0.5f / (threshold * threshold);
  const float invThresholdSqrt2PI = 0.3989422804014327f / threshold;
  const float cr = powf(in.ld(x, y, 0), inv_gamma), cg = powf(in.ld(x, y, 1), inv_gamma), cb = powf(in.ld(x, y, 2), inv_gamma);
  float z = 0.f, aR = 0.f, aG = 0.f, aB = 0.f;
  for (float dx = -radius; dx <= radius; dx += 1.f) {
    const float pt = sqrtf(radQ - dx * dx);
    for (float dy = -pt; dy <= pt; dy += 1.f) {
      const float bf = expf(-((dx * dx + dy * dy) * invSigmaQx2)) * invSigmaQx2PI;
      const int ix = static_cast<int>(static_cast<float>(x) + dx), iy = static_cast<int>(static_cast<float>(y) + dy);
      const float wr = in.ld(ix, iy, 0), wg = in.ld(ix, iy, 1), wb = in.ld(ix, iy, 2);
      const float dr = powf(wr, inv_gamma) - cr, dg = powf(wg, inv_gamma) - cg, db = powf(wb, inv_gamma) - cb;
      const float df = expf(-((dr * dr + dg * dg + db * db) * invThresholdSqx2)) * invThresholdSqrt2PI * bf;
      z += df;
      aR += df * wr; aG += df * wg; aB += df * wb;
    }
  }
  o[0] = aR / z; o[1] = aG / z; o[2] = aB / z; o[3] = 1.f;
}

// lut: int32 [4, 8192] (luma spatial, luma temporal, chroma spatial, chroma temporal)
__device__ __forceinline__ int hq_lowpass(const int* lut, int prev, int cur, int cls) {
  const int num = prev - cur;
  const int dt = num / 16;                           // C division truncates toward zero, as the shader's does
  const int idx = min(max(dt + 4096, 0), 8191);
  return cur + lut[cls * 8192 + idx];
}
__global__ void hqdn3d_kernel(Img in, float* out, const int* lut) {
  PIXEL_XY();
  const float r = in.ld(x, y, 0), g = in.ld(x, y, 1), b = in.ld(x, y, 2), a = in.ld(x, y, 3);
  // colour matrices evaluated in double, then rounded once (the CPU statement works on python floats here)
  const double rd = r, gd = g, bd = b;
  const float Y = clamp01(static_cast<float>(0.262700 * rd + 0.678000 * gd + 0.059300 * bd));
  const float U = clamp01(static_cast<float>(0.5 + (-0.139630 * rd + -0.360370 * gd + 0.500000 * bd)));
  const float V = clamp01(static_cast<float>(0.5 + (0.500000 * rd + -0.459786 * gd + -0.040214 * bd)));
  float res[3];
  const float src[3] = {Y, U, V};
  for (int c = 0; c < 3; ++c) {
    const int sp = c == 0 ? 0 : 2, tm = c == 0 ? 1 : 3;
    int pa = hq_lowpass(lut, 0, static_cast<int>(src[c] * 65535.0f) + 128, sp);
    pa = hq_lowpass(lut, 0, pa, sp);
    res[c] = static_cast<float>(hq_lowpass(lut, 0, pa, tm)) / 65535.0f;
  }
  const double yy = res[0], uu = static_cast<double>(res[1]) - 0.5, vv = static_cast<double>(res[2]) - 0.5;
  o[0] = clamp01(static_cast<float>(yy + 1.474600 * vv));
  o[1] = clamp01(static_cast<float>(yy + -0.164553 * uu + -0.571353 * vv));
  o[2] = clamp01(static_cast<float>(yy + 1.881400 * uu));
  o[3] = a;
}

// guided filter: moments -> box H -> box V (for both moment images) -> combine
__global__ void guided_moments_kernel(Img in, float* mI, float* mII) {
  const int x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= in.W || y >= in.H) return;
  const long long o = (static_cast<long long>(y) * in.W + x) * 4;
  for (int c = 0; c < 3; ++c) { const float v = in.ld(x, y, c); mI[o + c] = v; mII[o + c] = v * v; }
  mI[o + 3] = mII[o + 3] = in.ld(x, y, 3);
}
__global__ void box_kernel(Img in, float* out, int r, int vertical) {
  PIXEL_XY();
  const int anchor = r / 2;
  const float wv = 1.f / static_cast<float>(r);
  for (int c = 0; c < 4; ++c) {
    float acc = 0.f;
    for (int k = 0; k < r; ++k) acc += wv * (vertical ? in.ld(x, y - anchor + k, c) : in.ld(x - anchor + k, y, c));
    o[c] = acc;
  }
}
__global__ void guided_combine_kernel(Img in, const float* bmI, const float* bmII, float* out, float eps) {
  PIXEL_XY();
  const long long q = (static_cast<long long>(y) * in.W + x) * 4;
  for (int c = 0; c < 3; ++c) {
    const float mi = bmI[q + c], mii = bmII[q + c];
    const float var = mii - mi * mi;
    const float a = var / (var + eps);
    const float b = mi * (1.f - a);
    o[c] = clamp01(a * in.ld(x, y, c) + b);
  }
  o[3] = in.ld(x, y, 3);
}

__global__ void deband_kernel(Img in, float* out, float range, float direction, float threshold) {
  PIXEL_XY();
  // per-pixel pseudo-random offset; the sine is taken in double so the hash agrees with a CPU that does the same
  const float arg = static_cast<float>(x) * 12.9898f + static_cast<float>(y) * 78.233f;
  const float r = static_cast<float>(sin(static_cast<double>(arg))) * 43758.545f;
  const float fr = r - static_cast<float>(floor(static_cast<double>(r)));
  const float dirv = fr * direction;
  const int dist = static_cast<int>(fr * range);
  const int xp = static_cast<int>(static_cast<float>(cos(static_cast<double>(dirv))) * static_cast<float>(dist));
  const int yp = static_cast<int>(static_cast<float>(sin(static_cast<double>(dirv))) * static_cast<float>(dist));
  const int xr = min(max(x + xp, 0), in.W - 1), xl = min(max(x - xp, 0), in.W - 1);
  const int yP = min(max(y + yp, 0), in.H - 1), yM = min(max(y - yp, 0), in.H - 1);
  for (int c = 0; c < 3; ++c) {
    const float r0 = in.ld(xr, yP, c), r1 = in.ld(xr, yM, c), r2 = in.ld(xl, yM, c), r3 = in.ld(xl, yP, c), s = in.ld(x, y, c);
    const float avg = (r0 + r1 + r2 + r3) / 4.f;
    const bool flat = fabsf(s - r0) < threshold && fabsf(s - r1) < threshold && fabsf(s - r2) < threshold && fabsf(s - r3) < threshold;
    o[c] = flat ? avg : s;
  }
  o[3] = in.ld(x, y, 3);
}

// ---- colour group ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float cb_component(float v, float l, float s_in, float m_in, float h_in) {
  const float a = 4.f, b = 0.333f, scale = 0.7f;
  const float s = s_in * clamp01((b - l) * a + 0.5f) * scale;
  const float m = m_in * clamp01((l - b) * a + 0.5f) * clamp01((1.f - l - b) * a + 0.5f) * scale;
  const float h = h_in * clamp01((l + b - 1.f) * a + 0.5f) * scale;
  return clamp01(v + s + m + h);
}
struct CBParams { float s[3], m[3], h[3]; };
__global__ void colorbalance_kernel(Img in, float* out, CBParams p) {
  PIXEL_XY();
  const float r = in.ld(x, y, 0), g = in.ld(x, y, 1), b = in.ld(x, y, 2);
  const float l = fmaxf(r, fmaxf(g, b)) + fminf(r, fminf(g, b));
  o[0] = cb_component(r, l, p.s[0], p.m[0], p.h[0]);
  o[1] = cb_component(g, l, p.s[1], p.m[1], p.h[1]);
  o[2] = cb_component(b, l, p.s[2], p.m[2], p.h[2]);
  o[3] = in.ld(x, y, 3);
}
__global__ void cas_kernel(Img in, float* out, float strength) {
  PIXEL_XY();
  for (int c = 0; c < 3; ++c) {
    const float a = in.ld(x - 1, y - 1, c), b = in.ld(x, y - 1, c), cc = in.ld(x + 1, y - 1, c);
    const float d = in.ld(x - 1, y, c), e = in.ld(x, y, c), f = in.ld(x + 1, y, c);
    const float g = in.ld(x - 1, y + 1, c), h = in.ld(x, y + 1, c), i = in.ld(x + 1, y + 1, c);
    float mn = fminf(fminf(fminf(d, e), fminf(f, b)), h);
    const float mn2 = fminf(fminf(mn, fminf(a, cc)), fminf(g, i));
    mn += mn2;
    float mx = fmaxf(fmaxf(fmaxf(d, e), fmaxf(f, b)), h);
    const float mx2 = fmaxf(fmaxf(mx, fmaxf(a, cc)), fmaxf(g, i));
    mx += mx2;
    const float amp = sqrtf(clamp01(fminf(mn, 2.f - mx) / mx));
    const float w = amp / strength;
    o[c] = ((b + d + f + h) * w + e) / (1.f + 4.f * w);
  }
  o[3] = in.ld(x, y, 3);
}
struct Kern15 { float w[15]; };
__global__ void gauss_kernel(Img in, float* out, Kern15 k, int vertical) {
  PIXEL_XY();
  for (int c = 0; c < 4; ++c) {
    float acc = 0.f;
    for (int t = 0; t < 15; ++t) acc += k.w[t] * (vertical ? in.ld(x, y + t - 7, c) : in.ld(x + t - 7, y, c));
    o[c] = acc;
  }
}
__global__ void usm_combine_kernel(Img in, const float* blur, float* out, float amount, float threshold) {
  PIXEL_XY();
  const long long q = (static_cast<long long>(y) * in.W + x) * 4;
  for (int c = 0; c < 3; ++c) {
    const float orig = in.ld(x, y, c);
    const float diff = orig - blur[q + c];
    o[c] = clamp01(fabsf(diff) >= threshold ? orig + amount * diff : orig);
  }
  o[3] = in.ld(x, y, 3);
}
// lut: [N, N, N, 4] fp32, blue fastest
__global__ void lut3d_kernel(Img in, float* out, const float* lut, int N) {
  PIXEL_XY();
  const float sc = static_cast<float>(N - 1);
  const float fr = clamp01(in.ld(x, y, 0)) * sc, fg = clamp01(in.ld(x, y, 1)) * sc, fb = clamp01(in.ld(x, y, 2)) * sc;
  const int r0 = min(max(static_cast<int>(fr), 0), N - 2), g0 = min(max(static_cast<int>(fg), 0), N - 2), b0 = min(max(static_cast<int>(fb), 0), N - 2);
  const float dr = fr - r0, dg = fg - g0, db = fb - b0;
  for (int c = 0; c < 3; ++c) {
    auto L = [&](int ro, int go, int bo) { return lut[(((r0 + ro) * N + (g0 + go)) * N + (b0 + bo)) * 4 + c]; };
    const float c00 = L(0, 0, 0) * (1 - db) + L(0, 0, 1) * db, c01 = L(0, 1, 0) * (1 - db) + L(0, 1, 1) * db;
    const float c10 = L(1, 0, 0) * (1 - db) + L(1, 0, 1) * db, c11 = L(1, 1, 0) * (1 - db) + L(1, 1, 1) * db;
    const float c0 = c00 * (1 - dg) + c01 * dg, c1 = c10 * (1 - dg) + c11 * dg;
    o[c] = c0 * (1 - dr) + c1 * dr;
  }
  o[3] = in.ld(x, y, 3);
}

// ---- effects group ---------------------------------------------------------------------------------------------------------
#define UV()                                                            \
  float uvx = static_cast<float>(x) / static_cast<float>(in.W - 1);     \
  float uvy = static_cast<float>(y) / static_cast<float>(in.H - 1);
__device__ __forceinline__ int tex(float uv, int n) { return static_cast<int>(uv * static_cast<float>(n - 1)); }

__global__ void waterripple_kernel(Img in, float* out, float freq, float amount) {
  PIXEL_XY();
  UV();
  const float dx = uvx - 0.5f, dy = uvy - 0.5f;
  const float ln = sqrtf(dx * dx + dy * dy);
  const float fac = (amount * fabsf(sinf(ln * freq))) / ln;
  const int sx = tex(uvx + dx * fac, in.W), sy = tex(uvy + dy * fac, in.H);
  for (int c = 0; c < 4; ++c) o[c] = in.ld(sx, sy, c);
}
__device__ __forceinline__ float phase_progress(float progress_in, float duration, int shrink) {
  float p = gmod(progress_in, duration) / duration;
  if (shrink == 1 && p > 0.5f) p = 1.f - p;
  return p;
}
__global__ void soul_kernel(Img in, float* out, float progress_in, float duration, float max_scale, float max_alpha, int shrink) {
  PIXEL_XY();
  UV();
  const float p = phase_progress(progress_in, duration, shrink);
  const float alpha = max_alpha * (1.f - p);
  const float scale = 1.f + (max_scale - 1.f) * p;
  const int wx = tex(clamp01(0.5f + (uvx - 0.5f) / scale), in.W), wy = tex(clamp01(0.5f + (uvy - 0.5f) / scale), in.H);
  const int mx = tex(uvx, in.W), my = tex(uvy, in.H);
  for (int c = 0; c < 4; ++c) o[c] = in.ld(wx, wy, c) * (1.f - alpha) + in.ld(mx, my, c) * alpha;
}
__global__ void sway_kernel(Img in, float* out, float speed, float strength, float density, int horizontal) {
  PIXEL_XY();
  UV();
  const float wave = sinf((uvy + speed) * density) * strength / 1000.f;
  if (horizontal == 1) uvx += wave; else uvy += wave;
  const int sx = tex(clamp01(uvx), in.W), sy = tex(clamp01(uvy), in.H);
  for (int c = 0; c < 4; ++c) o[c] = in.ld(sx, sy, c);
}
__global__ void jitter_kernel(Img in, float* out, float progress_in, float duration, float max_scale, float offset, int shrink) {
  PIXEL_XY();
  UV();
  const float p = phase_progress(progress_in, duration, shrink);
  const float offc = offset * p;
  const float scale = 1.f + (max_scale - 1.f) * p;
  const float scx = clamp01(0.5f + (uvx - 0.5f) / scale), scy = clamp01(0.5f + (uvy - 0.5f) / scale);
  const int rx = tex(clamp01(scx + offc), in.W), ry = tex(clamp01(scy + offc), in.H);
  const int bx = tex(clamp01(scx - offc), in.W), by = tex(clamp01(scy - offc), in.H);
  const int mx = tex(scx, in.W), my = tex(scy, in.H);
  o[0] = in.ld(rx, ry, 0); o[1] = in.ld(mx, my, 1); o[2] = in.ld(bx, by, 2); o[3] = in.ld(mx, my, 3);
}

// star field
#define STAR_PI 3.1415f
__device__ __forceinline__ float star_random(float px_in, float py_in) {
  float px = gfract(px_in * 123.45f), py = gfract(py_in * 345.67f);
  const float d = (px * px + py * py) + 45.32f * (px + py);
  px += d; py += d;
  return gfract(px * py);
}
__device__ float star_core(float ux, float uy, float flaresize, float rot) {
  const float d = sqrtf(ux * ux + uy * uy);
  float core = 0.05f / d;
  const float ang = -2.f * STAR_PI * rot;
  float c = cosf(ang), s = sinf(ang);
  float nx = c * ux - s * uy, ny = s * ux + c * uy;
  ux = nx; uy = ny;
  core += fmaxf(1.f - fabsf(ux * uy * 3000.f), 0.f) * flaresize;
  const float ang2 = STAR_PI * 0.25f;
  c = cosf(ang2); s = sinf(ang2);
  nx = c * ux - s * uy; ny = s * ux + c * uy;
  core += fmaxf(1.f - fabsf(nx * ny * 3000.f), 0.f) * 0.3f * flaresize;
  return core * smoothstep(1.f, 0.05f, d);
}
__global__ void star_kernel(Img in, float* out, float progress, float speed, float layers, float red, float green, float blue) {
  PIXEL_XY();
  UV();
  const float delta_time = progress * speed * 0.01f, rot = progress * speed * 0.09f, stepi = 1.f / layers;
  const float col_p[3] = {red, green, blue};
  float col[3] = {0.f, 0.f, 0.f};
  float tx = uvx, ty = uvy;
  for (float i = 0.f; i < 1.f; i += stepi) {
    const float depth = gfract(i + delta_time);
    const float lscale = 64.f + (0.01f - 64.f) * depth;
    const float fader = depth * smoothstep(0.1f, 1.1f, depth);
    const float loff = i * (3430.00f + gfract(i));
    const float ang = rot * i * -10.f;
    const float c = cosf(ang), s = sinf(ang);
    const float ntx = c * tx - s * ty, nty = s * tx + c * ty;
    tx = ntx; ty = nty;
    const float sfx = tx * lscale + loff, sfy = ty * lscale + loff;
    const float gvx = gfract(sfx) - 0.5f, gvy = gfract(sfy) - 0.5f, idx = gfloor(sfx), idy = gfloor(sfy);
    float lc[3] = {0.f, 0.f, 0.f};
    for (int yy = -1; yy <= 1; ++yy)
      for (int xx = -1; xx <= 1; ++xx) {
        const float ox = static_cast<float>(xx), oy = static_cast<float>(yy);
        const float rn = star_random(idx + ox, idy + oy);
        const float rpx = gvx - ox - (rn - 0.5f), rpy = gvy - oy - (gfract(rn * 45.f) - 0.5f);
        const float size = gfract(rn * 1356.33f);
        const float st = star_core(rpx, rpy, smoothstep(0.9f, 1.f, size), rot);
        const float seed = gfract(rn * 2150.f) * (3.f * STAR_PI) * progress;
        const float m = 0.4f * sinf(progress);
        const float dim = 15.f / layers;
        for (int k = 0; k < 3; ++k) {
          float cc = sinf(col_p[k] * seed) * m + 0.6f;
          cc = cc * (k == 2 ? col_p[k] + size : col_p[k]);
          lc[k] += st * size * cc * dim;
        }
      }
    for (int k = 0; k < 3; ++k) col[k] += lc[k] * fader;
  }
  for (int k = 0; k < 3; ++k) o[k] = in.ld(x, y, k) + col[k];
  o[3] = in.ld(x, y, 3);
}

// lighting: hue rotation + value lift in HSV, saturation lift in HSL, blend towards white
__device__ __forceinline__ void rgb2hcv(float r, float g, float b, float& h, float& c, float& v) {
  float px, py, pz, pw;
  if (g < b) { px = b; py = g; pz = -1.f; pw = 2.f / 3.f; } else { px = g; py = b; pz = 0.f; pw = -1.f / 3.f; }
  float qx, qy, qz, qw;
  if (r < px) { qx = px; qy = py; qz = pw; qw = r; } else { qx = r; qy = py; qz = pz; qw = px; }
  c = qx - fminf(qw, qy);
  h = fabsf((qw - qy) / (6.f * c + 1.0e-10f) + qz);
  v = qx;
}
__global__ void lighting_kernel(Img in, float* out, float progress_in, float duration, float saturation, float light) {
  PIXEL_XY();
  const float p = gmod(progress_in, duration) / duration;
  const float hue = fabsf(sinf(p * (3.1415926f / duration))) * 360.f / 360.f;
  const float r = in.ld(x, y, 0), g = in.ld(x, y, 1), b = in.ld(x, y, 2);
  float fh, c, fv;
  rgb2hcv(r, g, b, fh, c, fv);
  const float fs = c / (fv + 1.0e-10f);
  fh += hue;
  fv = clamp01(fv + saturation / 10.f);
  float m[3];
  const float K[3] = {1.f, 2.f / 3.f, 1.f / 3.f};
  for (int k = 0; k < 3; ++k) m[k] = fv * ((1.f - fs) + clamp01(fabsf(gfract(fh + K[k]) * 6.f - 3.f) - 1.f) * fs);
  float lh, lc, lv;
  rgb2hcv(m[0], m[1], m[2], lh, lc, lv);
  const float z = lv - lc * 0.5f;
  float ls = lc / (1.f - fabsf(2.f * z - 1.f) + 1.0e-10f);
  ls = clamp01(ls + saturation * 0.5f);
  const float hr = clamp01(fabsf(lh * 6.f - 3.f) - 1.f), hg = clamp01(2.f - fabsf(lh * 6.f - 2.f)), hb = clamp01(2.f - fabsf(lh * 6.f - 4.f));
  const float cc = (1.f - fabsf(2.f * z - 1.f)) * ls;
  const float rgb[3] = {(hr - 0.5f) * cc + z, (hg - 0.5f) * cc + z, (hb - 0.5f) * cc + z};
  for (int k = 0; k < 3; ++k) o[k] = rgb[k] * (1.f - light) + 1.f * light;
  o[3] = in.ld(x, y, 3);
}

}  // namespace filt
}  // namespace mdb

using namespace mdb::filt;

// op codes: 0 smartdenoise, 1 hqdn3d, 2 guided, 3 deband, 4 colorbalance, 5 cas, 6 usm, 7 lut3d, 8 waterripple, 9 soul,
// 10 sway, 11 star, 12 lighting, 13 jitter. params: fp32 host array (meaning per op, see ops/filters.py); aux: device
// pointer (hqdn3d: int32 lut [4, 8192]; lut3d: fp32 [N, N, N, 4] with N = params[0]); tmp: device scratch of
// 4 * H * W * 4 floats (guided) or 2 * ... (usm), may be null for single-pass filters.
extern "C" int mdb_image_filter(int op, const float* in_p, float* out, float* tmp, int H, int W, const float* pr, int np,
                                const void* aux, cudaStream_t st) {
  if (H <= 0 || W <= 0) return 0;
  if (H < 2 || W < 2) return -1;
  Img in{in_p, H, W};
  const dim3 blk(16, 16), grd((W + 15) / 16, (H + 15) / 16);
  const long long n4 = static_cast<long long>(H) * W * 4;
  auto need = [&](int n) { return np >= n; };
  switch (op) {
    case 0: if (!need(3)) return -2; smartdenoise_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], pr[1], pr[2]); break;
    case 1: if (!aux) return -3; hqdn3d_kernel<<<grd, blk, 0, st>>>(in, out, static_cast<const int*>(aux)); break;
    case 2: {
      if (!need(2) || !tmp) return -2;
      float *mI = tmp, *mII = tmp + n4, *t0 = tmp + 2 * n4, *t1 = tmp + 3 * n4;
      const int r = static_cast<int>(pr[0]);
      if (r < 1 || r > 64) return -2;
      guided_moments_kernel<<<grd, blk, 0, st>>>(in, mI, mII);
      box_kernel<<<grd, blk, 0, st>>>(Img{mI, H, W}, t0, r, 0);
      box_kernel<<<grd, blk, 0, st>>>(Img{t0, H, W}, mI, r, 1);
      box_kernel<<<grd, blk, 0, st>>>(Img{mII, H, W}, t1, r, 0);
      box_kernel<<<grd, blk, 0, st>>>(Img{t1, H, W}, mII, r, 1);
      guided_combine_kernel<<<grd, blk, 0, st>>>(in, mI, mII, out, pr[1]);
      break;
    }
    case 3: if (!need(3)) return -2; deband_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], pr[1], pr[2]); break;
    case 4: {
      if (!need(9)) return -2;
      CBParams p;
      for (int i = 0; i < 3; ++i) { p.s[i] = pr[i]; p.m[i] = pr[3 + i]; p.h[i] = pr[6 + i]; }
      colorbalance_kernel<<<grd, blk, 0, st>>>(in, out, p);
      break;
    }
    case 5: if (!need(1)) return -2; cas_kernel<<<grd, blk, 0, st>>>(in, out, pr[0]); break;
    case 6: {
      if (!need(17) || !tmp) return -2;              // amount, threshold, 15 gaussian taps
      Kern15 k;
      for (int i = 0; i < 15; ++i) k.w[i] = pr[2 + i];
      gauss_kernel<<<grd, blk, 0, st>>>(in, tmp, k, 0);
      gauss_kernel<<<grd, blk, 0, st>>>(Img{tmp, H, W}, tmp + n4, k, 1);
      usm_combine_kernel<<<grd, blk, 0, st>>>(in, tmp + n4, out, pr[0], pr[1]);
      break;
    }
    case 7: if (!need(1) || !aux || pr[0] < 2) return -2; lut3d_kernel<<<grd, blk, 0, st>>>(in, out, static_cast<const float*>(aux), static_cast<int>(pr[0])); break;
    case 8: if (!need(2)) return -2; waterripple_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], pr[1]); break;
    case 9: if (!need(5)) return -2; soul_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], 1.f / pr[1], pr[2], pr[3], static_cast<int>(pr[4])); break;
    case 10: if (!need(4)) return -2; sway_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], pr[1], pr[2], static_cast<int>(pr[3])); break;
    case 11: if (!need(6) || pr[2] < 1.f) return -2; star_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], pr[1], pr[2], pr[3], pr[4], pr[5]); break;
    case 12: if (!need(4)) return -2; lighting_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], 1.f / pr[1], pr[2], pr[3]); break;
    case 13: if (!need(5)) return -2; jitter_kernel<<<grd, blk, 0, st>>>(in, out, pr[0], 1.f / pr[1], pr[2], pr[3], static_cast<int>(pr[4])); break;
    default: return -4;
  }
  return static_cast<int>(cudaGetLastError());
}
