// NHWC image kernels around the implicit-GEMM convolution: GroupNorm fused with SiLU, nearest 2x upsample,
// pixel shuffle / unshuffle, 2x2 average pool. 128-bit accesses, fp32 statistics.
//
// Reference behaviour: serenitymojo/ops/norm.mojo:855-1049 (NHWC GroupNorm(32)), serenitymojo/models/vae/upsample.mojo
// (nearest 2x), serenitymojo/ops/pixelshuffle.mojo:144-770, serenitymojo/models/vae/decoder2d.mojo:150-362 (how the
// ResnetBlock uses GN -> SiLU -> conv).
#include "common.cuh"
#include "kernels_api.h"

namespace mdb {

// stats[n, g] = (mean, rstd) over H*W*(C/G) elements. One block per (n, g).
__global__ void __launch_bounds__(256)
group_norm_stats_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ stats, int HW, int C, int G, float eps) {
  const int n = blockIdx.x / G, g = blockIdx.x % G;
  const int cpg = C / G;
  const __nv_bfloat16* base = x + static_cast<size_t>(n) * HW * C + g * cpg;
  const int vec = cpg >> 3;  // cpg is a multiple of 8 on the vector path, else scalar
  float s = 0.f, ss = 0.f;
  if (vec > 0 && (cpg & 7) == 0) {
    const long long total = static_cast<long long>(HW) * vec;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) {
      const int p = static_cast<int>(i / vec), v = static_cast<int>(i % vec);
      const uint4 u = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(p) * C + v * 8);
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(w4[k]);
        s += f.x + f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
  } else {
    const long long total = static_cast<long long>(HW) * cpg;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) {
      const float f = __bfloat162float(base[(i / cpg) * C + (i % cpg)]);
      s += f;
      ss += f * f;
    }
  }
  __shared__ float rs[8], rss[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  }
  if ((threadIdx.x & 31) == 0) {
    rs[threadIdx.x >> 5] = s;
    rss[threadIdx.x >> 5] = ss;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int i = 0; i < 8; ++i) {
      a += rs[i];
      b += rss[i];
    }
    const float cnt = static_cast<float>(HW) * cpg;
    const float mean = a / cnt;
    const float var = fmaxf(b / cnt - mean * mean, 0.f);
    stats[2 * blockIdx.x] = mean;
    stats[2 * blockIdx.x + 1] = rsqrtf(var + eps);
  }
}

// Statistics over many blocks: a block takes a range of pixels of one sample for ALL channels (each thread owns one
// 8-channel vector and strides over the pixels: 128-bit coalesced loads). Its per-channel partials are reduced in a fixed
// order (over the pixel lanes, then over the channels of a group) and written to part[n, chunk, g] = (sum, sum of squares);
// a second kernel adds the chunks in order and turns them into (mean, rstd). No atomics: the result does not depend on
// scheduling. One block per (sample, group), as the kernel above, leaves most of the device idle for a 1024 x 1024 x 128
// image (32 blocks, and 4 channels per group defeat its vector path).
__global__ void __launch_bounds__(256)
group_norm_partial_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, int HW, int C, int G, int ppb) {
  extern __shared__ float gsm[];                 // [256][16] per-thread channel partials, then [C][2] channel sums
  const int n = blockIdx.y, cv = C >> 3, cpg = C / G;
  const int lanes = blockDim.x / cv;
  float s[8], ss[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) s[k] = ss[k] = 0.f;
  if (static_cast<int>(threadIdx.x) < lanes * cv) {
    const int v = threadIdx.x % cv, pl = threadIdx.x / cv;
    const int p0 = blockIdx.x * ppb, p1 = min(p0 + ppb, HW);
    const __nv_bfloat16* base = x + (static_cast<size_t>(n) * HW) * C + v * 8;
    for (int p = p0 + pl; p < p1; p += lanes) {
      const uint4 u = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(p) * C);
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(w4[k]);
        s[2 * k] += f.x; ss[2 * k] += f.x * f.x;
        s[2 * k + 1] += f.y; ss[2 * k + 1] += f.y * f.y;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) { gsm[threadIdx.x * 16 + k] = s[k]; gsm[threadIdx.x * 16 + 8 + k] = ss[k]; }
  __syncthreads();
  float* csum = gsm + 256 * 16;                  // [C][2]
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int v = c >> 3, k = c & 7;
    float a = 0.f, b = 0.f;
    for (int pl = 0; pl < lanes; ++pl) { a += gsm[(pl * cv + v) * 16 + k]; b += gsm[(pl * cv + v) * 16 + 8 + k]; }
    csum[2 * c] = a; csum[2 * c + 1] = b;
  }
  __syncthreads();
  float* out = part + (static_cast<size_t>(n) * gridDim.x + blockIdx.x) * 2 * G;
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    float a = 0.f, b = 0.f;
    for (int c = g * cpg; c < (g + 1) * cpg; ++c) { a += csum[2 * c]; b += csum[2 * c + 1]; }
    out[2 * g] = a; out[2 * g + 1] = b;
  }
}
// stats[n, g] = (mean, rstd) (or, with cnt <= 0, the raw sums) from the chunk partials, added in chunk order
__global__ void group_norm_finalize_kernel(const float* __restrict__ part, float* __restrict__ stats, int N, int G, int chunks, int stride,
                                           float cnt, float eps) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * G) return;
  const int n = i / G, g = i % G;
  float a = 0.f, b = 0.f;
  for (int c = 0; c < chunks; ++c) {
    const float* p = part + (static_cast<size_t>(n) * chunks + c) * stride + 2 * g;
    a += p[0]; b += p[1];
  }
  if (cnt > 0.f) {
    const float mean = a / cnt;
    const float var = fmaxf(b / cnt - mean * mean, 0.f);
    stats[2 * i] = mean;
    stats[2 * i + 1] = rsqrtf(var + eps);
  } else {
    stats[2 * i] = a;
    stats[2 * i + 1] = b;
  }
}

// y = act((x - mean) * rstd * w[c] + b[c]); act 0 none, 2 SiLU
__global__ void group_norm_apply_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                        const float* __restrict__ stats, const __nv_bfloat16* __restrict__ w,
                                        const __nv_bfloat16* __restrict__ b, long long total_vec, int HW, int C, int G,
                                        int act) {
  const int cv = C >> 3, cpg = C / G;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_vec; i += (long long)gridDim.x * blockDim.x) {
    const int c0 = static_cast<int>(i % cv) * 8;
    const long long pix = i / cv;
    const int n = static_cast<int>(pix / HW);
    const uint4 u = *reinterpret_cast<const uint4*>(x + i * 8);
    const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
    float v[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w4[k]);
      v[2 * k] = f.x;
      v[2 * k + 1] = f.y;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = c0 + k;
      const int g = c / cpg;
      const float mean = stats[2 * (n * G + g)], rstd = stats[2 * (n * G + g) + 1];
      float t = (v[k] - mean) * rstd;
      if (w) t = t * __bfloat162float(w[c]) + (b ? __bfloat162float(b[c]) : 0.f);
      if (act == 2) t = silu_f(t);
      v[k] = t;
    }
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]);
    o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(y + i * 8) = o;
  }
}

// ---- GroupNorm backward -------------------------------------------------------------------------------------------------
// With xh = (x - mean) * rstd, z = xh * w + b, y = act(z) and g = dy * act'(z) * w:
//   dx = rstd * (g - mean_group(g) - xh * mean_group(g * xh)),   dw[c] = sum dy act'(z) xh,   db[c] = sum dy act'(z)
// (serenitymojo/ops/norm_backward.mojo:951,1080). Pass 1 (one block per sample and group) forms the two group means and,
// when asked, adds the per-channel sums into fp32 dw / db; pass 2 is elementwise.
__device__ __forceinline__ float gn_dact(float z, int act) {
  if (act != 2) return 1.f;
  const float sg = 1.f / (1.f + __expf(-z));
  return sg * (1.f + z * (1.f - sg));
}
__global__ void __launch_bounds__(256)
group_norm_bwd_sums_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ stats,
                           const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b, float* __restrict__ sums,
                           float* __restrict__ dw, float* __restrict__ db, int HW, int C, int G, int act) {
  const int n = blockIdx.x / G, g = blockIdx.x % G;
  const int cpg = C / G;
  const size_t base = static_cast<size_t>(n) * HW * C + g * cpg;
  const float mean = stats[2 * blockIdx.x], rstd = stats[2 * blockIdx.x + 1];
  float s1 = 0.f, s2 = 0.f;
  // each thread keeps to one channel of the group while it walks the pixels, so its dw / db partials are per channel;
  // blockDim / cpg pixel lanes per channel, the threads beyond lanes * cpg idle
  const int lanes = blockDim.x / cpg;
  if (static_cast<int>(threadIdx.x) < lanes * cpg) {
    const int c = threadIdx.x % cpg, pl = threadIdx.x / cpg;
    const float wc = w ? __bfloat162float(w[g * cpg + c]) : 1.f, bc = b ? __bfloat162float(b[g * cpg + c]) : 0.f;
    float a1 = 0.f, a2 = 0.f;
    for (int p = pl; p < HW; p += lanes) {
      const size_t off = base + static_cast<size_t>(p) * C + c;
      const float xh = (__bfloat162float(x[off]) - mean) * rstd;
      const float dz = __bfloat162float(dy[off]) * gn_dact(xh * wc + bc, act);
      a1 += dz;
      a2 += dz * xh;
    }
    if (dw) atomicAdd(&dw[g * cpg + c], a2);
    if (db) atomicAdd(&db[g * cpg + c], a1);
    s1 = a1 * wc;
    s2 = a2 * wc;
  }
  __shared__ float r1[8], r2[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if ((threadIdx.x & 31) == 0) { r1[threadIdx.x >> 5] = s1; r2[threadIdx.x >> 5] = s2; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, c2 = 0.f;
    for (int i = 0; i < 8; ++i) { a += r1[i]; c2 += r2[i]; }
    const float cnt = static_cast<float>(HW) * cpg;
    sums[2 * blockIdx.x] = a / cnt;
    sums[2 * blockIdx.x + 1] = c2 / cnt;
  }
}
// many-block form of the sums above (same decomposition and ordered reductions as group_norm_partial_kernel). part[n, chunk]
// holds per group (sum g, sum g * xh) and, when weight gradients are wanted, per channel (sum dz * xh, sum dz) after the
// 2 * G group values; group_norm_finalize_kernel / group_norm_wgrad_kernel add the chunks in order.
__global__ void __launch_bounds__(256)
group_norm_bwd_partial_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ stats,
                              const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b, float* __restrict__ part,
                              int wgrad, int HW, int C, int G, int act, int ppb) {
  extern __shared__ float gsm[];                 // [256][16], then [C][2]
  const int n = blockIdx.y, cv = C >> 3, cpg = C / G;
  const int lanes = blockDim.x / cv;
  float a1[8], a2[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a1[k] = a2[k] = 0.f;
  if (static_cast<int>(threadIdx.x) < lanes * cv) {
    const int v = threadIdx.x % cv, pl = threadIdx.x / cv;
    const int p0 = blockIdx.x * ppb, p1 = min(p0 + ppb, HW);
    float wc[8], bc[8], mean[8], rstd[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = v * 8 + k, g = c / cpg;
      wc[k] = w ? __bfloat162float(w[c]) : 1.f;
      bc[k] = b ? __bfloat162float(b[c]) : 0.f;
      mean[k] = stats[2 * (n * G + g)];
      rstd[k] = stats[2 * (n * G + g) + 1];
    }
    const size_t base = (static_cast<size_t>(n) * HW) * C + v * 8;
    for (int p = p0 + pl; p < p1; p += lanes) {
      const uint4 ux = *reinterpret_cast<const uint4*>(x + base + static_cast<size_t>(p) * C);
      const uint4 ud = *reinterpret_cast<const uint4*>(dy + base + static_cast<size_t>(p) * C);
      const uint32_t x4[4] = {ux.x, ux.y, ux.z, ux.w}, d4[4] = {ud.x, ud.y, ud.z, ud.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float2 fx = unpack_bf16x2(x4[k >> 1]), fd = unpack_bf16x2(d4[k >> 1]);
        const float xh = (((k & 1) ? fx.y : fx.x) - mean[k]) * rstd[k];
        const float dz = ((k & 1) ? fd.y : fd.x) * gn_dact(xh * wc[k] + bc[k], act);
        a1[k] += dz;
        a2[k] += dz * xh;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) { gsm[threadIdx.x * 16 + k] = a1[k]; gsm[threadIdx.x * 16 + 8 + k] = a2[k]; }
  __syncthreads();
  float* csum = gsm + 256 * 16;                  // [C][2] = (sum dz, sum dz * xh)
  const int stride = 2 * G + (wgrad ? 2 * C : 0);
  float* out = part + (static_cast<size_t>(n) * gridDim.x + blockIdx.x) * stride;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int v = c >> 3, k = c & 7;
    float a = 0.f, bsum = 0.f;
    for (int pl = 0; pl < lanes; ++pl) { a += gsm[(pl * cv + v) * 16 + k]; bsum += gsm[(pl * cv + v) * 16 + 8 + k]; }
    csum[2 * c] = a; csum[2 * c + 1] = bsum;
    if (wgrad) { out[2 * G + 2 * c] = bsum; out[2 * G + 2 * c + 1] = a; }
  }
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    float a = 0.f, bsum = 0.f;
    for (int c = g * cpg; c < (g + 1) * cpg; ++c) {
      const float wc = w ? __bfloat162float(w[c]) : 1.f;
      a += csum[2 * c] * wc; bsum += csum[2 * c + 1] * wc;
    }
    out[2 * g] = a; out[2 * g + 1] = bsum;
  }
}
// dw[c] / db[c] += over samples and chunks, in order
__global__ void group_norm_wgrad_kernel(const float* __restrict__ part, float* __restrict__ dw, float* __restrict__ db, int N, int C, int G,
                                        int chunks) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int stride = 2 * G + 2 * C;
  float a = 0.f, b = 0.f;
  for (int i = 0; i < N * chunks; ++i) { a += part[static_cast<size_t>(i) * stride + 2 * G + 2 * c]; b += part[static_cast<size_t>(i) * stride + 2 * G + 2 * c + 1]; }
  dw[c] += a;
  db[c] += b;
}
__global__ void group_norm_bwd_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                            __nv_bfloat16* __restrict__ dx, const float* __restrict__ stats, const float* __restrict__ sums,
                                            const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b, long long total_vec,
                                            int HW, int C, int G, int act, float sum_scale) {
  const int cv = C >> 3, cpg = C / G;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_vec; i += (long long)gridDim.x * blockDim.x) {
    const int c0 = static_cast<int>(i % cv) * 8;
    const int n = static_cast<int>((i / cv) / HW);
    const uint4 ux = *reinterpret_cast<const uint4*>(x + i * 8), ud = *reinterpret_cast<const uint4*>(dy + i * 8);
    const uint32_t x4[4] = {ux.x, ux.y, ux.z, ux.w}, d4[4] = {ud.x, ud.y, ud.z, ud.w};
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float2 fx = unpack_bf16x2(x4[k >> 1]), fd = unpack_bf16x2(d4[k >> 1]);
      const float xv = (k & 1) ? fx.y : fx.x, dv = (k & 1) ? fd.y : fd.x;
      const int c = c0 + k, g = c / cpg;
      const float mean = stats[2 * (n * G + g)], rstd = stats[2 * (n * G + g) + 1];
      const float m1 = sums[2 * (n * G + g)] * sum_scale, m2 = sums[2 * (n * G + g) + 1] * sum_scale;
      const float wc = w ? __bfloat162float(w[c]) : 1.f, bc = b ? __bfloat162float(b[c]) : 0.f;
      const float xh = (xv - mean) * rstd;
      const float gg = dv * gn_dact(xh * wc + bc, act) * wc;
      v[k] = rstd * (gg - m1 - xh * m2);
    }
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]); o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(dx + i * 8) = o;
  }
}

// nearest-neighbour 2x upsample, NHWC
__global__ void upsample2x_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int N, int H, int W, int cv) {
  const long long total = static_cast<long long>(N) * H * 2 * W * 2 * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = static_cast<int>(i % cv);
    long long r = i / cv;
    const int ow = static_cast<int>(r % (2 * W));
    r /= 2 * W;
    const int oh = static_cast<int>(r % (2 * H));
    const int n = static_cast<int>(r / (2 * H));
    y[i] = x[((static_cast<long long>(n) * H + (oh >> 1)) * W + (ow >> 1)) * cv + c];
  }
}

// 2x2 average pool, NHWC (down-sampling path of encoders when no strided conv is used)
__global__ void avgpool2x_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int N, int H, int W,
                                 int C) {
  const int Ho = H / 2, Wo = W / 2;
  const long long total = static_cast<long long>(N) * Ho * Wo * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = static_cast<int>(i % C);
    long long r = i / C;
    const int ow = static_cast<int>(r % Wo);
    r /= Wo;
    const int oh = static_cast<int>(r % Ho);
    const int n = static_cast<int>(r / Ho);
    const __nv_bfloat16* p = x + ((static_cast<long long>(n) * H + 2 * oh) * W + 2 * ow) * C + c;
    const float s = __bfloat162float(p[0]) + __bfloat162float(p[C]) + __bfloat162float(p[static_cast<long long>(W) * C]) +
                    __bfloat162float(p[static_cast<long long>(W) * C + C]);
    y[i] = __float2bfloat16_rn(0.25f * s);
  }
}

static inline int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = static_cast<long long>(mdb::device_sm_count()) * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace mdb

using namespace mdb;
typedef __nv_bfloat16 bf16;

// How the many-block kernels split a sample: chunk count and pixels per chunk (0 chunks: use the block-per-group kernels)
static void gn_chunks(int N, int HW, int C, int G, int* chunks, int* ppb) {
  const int cv = C / 8, sms = mdb::device_sm_count();
  *chunks = 0;
  *ppb = 0;
  if (cv > 256 || C > 2048 || N * G >= 4 * sms) return;
  int ch = (4 * sms + N - 1) / N;                               // about four blocks per SM over all samples
  int pp = (HW + ch - 1) / ch;
  const int lanes = 256 / cv;
  if (pp < 4 * lanes) pp = 4 * lanes;                           // at least a few pixels per thread
  *ppb = pp;
  *chunks = (HW + pp - 1) / pp;
}
// fp32 elements of scratch the forward (wgrad < 0) or the backward (wgrad 0 / 1) needs
extern "C" long long mdb_group_norm_scratch_floats(int N, int HW, int C, int G, int wgrad) {
  int chunks, ppb;
  gn_chunks(N, HW, C, G, &chunks, &ppb);
  const long long base = (wgrad < 0 ? 2ll : 4ll) * N * G;
  const long long fwd = 2ll * G * N * chunks;
  const long long bwd = (2ll * G + (wgrad > 0 ? 2ll * C : 0)) * N * chunks;
  return base + (wgrad < 0 ? fwd : (fwd > bwd ? fwd : bwd));
}
// (mean, rstd) per (sample, group) into stats; ``part`` is scratch for the chunk partials
static int launch_group_stats(const void* x, float* stats, float* part, int N, int HW, int C, int G, float eps, cudaStream_t st) {
  int chunks, ppb;
  gn_chunks(N, HW, C, G, &chunks, &ppb);
  if (chunks == 0) {
    group_norm_stats_kernel<<<N * G, 256, 0, st>>>((const bf16*)x, stats, HW, C, G, eps);
    return (int)cudaGetLastError();
  }
  const size_t smem = (256 * 16 + 2 * C) * sizeof(float);
  group_norm_partial_kernel<<<dim3(chunks, N), 256, smem, st>>>((const bf16*)x, part, HW, C, G, ppb);
  group_norm_finalize_kernel<<<(N * G + 255) / 256, 256, 0, st>>>(part, stats, N, G, chunks, 2 * G, static_cast<float>(HW) * (C / G), eps);
  return (int)cudaGetLastError();
}

// stats: [N * G, 2] scratch (mean, rstd), sums: [N * G, 2] scratch; dw / db: fp32 [C] accumulators (zeroed by the caller) or null
extern "C" int mdb_group_norm_bwd(const void* x, const void* dy, void* dx, float* scratch, const void* w, const void* b, float* dw,
                                  float* db, int N, int HW, int C, int G, float eps, int act, cudaStream_t st) {
  if (C % G || C % 8 || (act != 0 && act != 2) || (C / G) > 256) return -1;
  if (N == 0) return 0;
  float* stats = scratch;
  float* sums = scratch + 2ll * N * G;
  float* part = scratch + 4ll * N * G;
  if (int rc = launch_group_stats(x, stats, part, N, HW, C, G, eps, st)) return rc;
  int chunks, ppb;
  gn_chunks(N, HW, C, G, &chunks, &ppb);
  if (chunks == 0) {
    group_norm_bwd_sums_kernel<<<N * G, 256, 0, st>>>((const bf16*)x, (const bf16*)dy, stats, (const bf16*)w, (const bf16*)b, sums, dw, db,
                                                      HW, C, G, act);
  } else {
    const int wgrad = dw != nullptr ? 1 : 0;
    const size_t smem = (256 * 16 + 2 * C) * sizeof(float);
    group_norm_bwd_partial_kernel<<<dim3(chunks, N), 256, smem, st>>>((const bf16*)x, (const bf16*)dy, stats, (const bf16*)w, (const bf16*)b,
                                                                      part, wgrad, HW, C, G, act, ppb);
    if (wgrad) group_norm_wgrad_kernel<<<(C + 255) / 256, 256, 0, st>>>(part, dw, db, N, C, G, chunks);
    // raw group sums (cnt <= 0), chunks added in order
    group_norm_finalize_kernel<<<(N * G + 255) / 256, 256, 0, st>>>(part, sums, N, G, chunks, 2 * G + (wgrad ? 2 * C : 0), -1.f, 0.f);
  }
  const float sum_scale = chunks == 0 ? 1.f : 1.f / (static_cast<float>(HW) * (C / G));
  const long long tv = static_cast<long long>(N) * HW * (C / 8);
  group_norm_bwd_apply_kernel<<<grid_for(tv, 256), 256, 0, st>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, stats, sums, (const bf16*)w,
                                                                 (const bf16*)b, tv, HW, C, G, act, sum_scale);
  return (int)cudaGetLastError();
}
extern "C" int mdb_group_norm(const void* x, void* y, float* stats, const void* w, const void* b, int N, int HW, int C,
                              int G, float eps, int act, cudaStream_t st) {
  if (C % 8 || C % G) return -1;
  if (N <= 0 || HW <= 0) return 0;
  if (int rc = launch_group_stats(x, stats, stats + 2ll * N * G, N, HW, C, G, eps, st)) return rc;
  const long long tv = static_cast<long long>(N) * HW * (C / 8);
  group_norm_apply_kernel<<<grid_for(tv, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, stats, (const bf16*)w,
                                                             (const bf16*)b, tv, HW, C, G, act);
  return (int)cudaGetLastError();
}
extern "C" int mdb_upsample2x(const void* x, void* y, int N, int H, int W, int C, cudaStream_t st) {
  if (C % 8) return -1;
  const long long total = static_cast<long long>(N) * H * W * 4 * (C / 8);
  if (total <= 0) return 0;
  upsample2x_kernel<<<grid_for(total, 256), 256, 0, st>>>((const uint4*)x, (uint4*)y, N, H, W, C / 8);
  return (int)cudaGetLastError();
}
extern "C" int mdb_avgpool2x(const void* x, void* y, int N, int H, int W, int C, cudaStream_t st) {
  const long long total = static_cast<long long>(N) * (H / 2) * (W / 2) * C;
  if (total <= 0) return 0;
  avgpool2x_kernel<<<grid_for(total, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, N, H, W, C);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------
// GroupNorm with a built-in workspace (see the declaration for the contract a caller relies on).
// The statistics buffer is a file-scope device array, so the address is fixed for the life of the module on each device
// and the call has nothing to allocate or free.
// ---------------------------------------------------------------------------------------------------------------
#include <cstdio>

static __device__ __align__(256) float g_group_norm_static_stats[2 * MDB_GROUP_NORM_STATIC_MAX_GROUPS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_stats_addr[kMaxDevices];   // per device; written once, always with the same value for that device

// Address of the array on the current device. cudaGetSymbolAddress answers for whichever device is current, so the
// cache is indexed by device ordinal. Two threads that get here together store the same pointer.
int static_stats_ptr(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -21;
  float* p = g_static_stats_addr[dev];
  if (p == nullptr) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_group_norm_static_stats);
    if (e != cudaSuccess) return static_cast<int>(e);
    p = static_cast<float*>(sym);
    g_static_stats_addr[dev] = p;
  }
  *out = p;
  return 0;
}
}  // namespace

extern "C" int mdb_group_norm_static_ws(const void* x, void* y, const void* w, const void* b, int N, int HW, int C,
                                        int G, float eps, int act, cudaStream_t st) {
  if (G <= 0 || C <= 0 || C % 8 || C % G) return -1;
  if (N <= 0 || HW <= 0) return 0;
  const long long groups = static_cast<long long>(N) * G;
  if (groups > MDB_GROUP_NORM_STATIC_MAX_GROUPS) {
    fprintf(stderr,
            "mdb_group_norm_static_ws: N * G = %lld exceeds the built-in workspace of %d (sample, group) pairs; "
            "split the batch or call mdb_group_norm with a buffer of your own\n",
            groups, MDB_GROUP_NORM_STATIC_MAX_GROUPS);
    return MDB_ERR_STATIC_WS_TOO_SMALL;
  }
  float* stats = nullptr;
  const int rc = static_stats_ptr(&stats);
  if (rc) return rc;
  // same two launches as mdb_group_norm; the first fills stats[0 .. 2 * N * G), the second reads exactly that range
  group_norm_stats_kernel<<<N * G, 256, 0, st>>>((const bf16*)x, stats, HW, C, G, eps);
  const long long tv = static_cast<long long>(N) * HW * (C / 8);
  group_norm_apply_kernel<<<grid_for(tv, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, stats, (const bf16*)w,
                                                             (const bf16*)b, tv, HW, C, G, act);
  return (int)cudaGetLastError();
}
