// Row kernels for sm_100a: LayerNorm / RMSNorm fused with adaLN modulation (forward and dx backward),
// and per-head QK-RMSNorm fused with rotary embedding applied in place on a packed qkv buffer.
// All loads and stores are 128-bit; statistics are fp32; a row stays in registers between the
// reduction and the write, so each element crosses HBM exactly once per direction.
//
// Reference behaviour matched: serenitymojo/ops/norm.mojo:47-230 (rms_norm), :318-460,652-782 (layer_norm,
// no-affine), serenitymojo/ops/elementwise.mojo:38-105 (modulate), serenitymojo/ops/rope.mojo:41-279
// (interleaved and half-split rotation), serenitymojo/ops/norm_backward.mojo:59-208,
// serenitymojo/ops/rope_struct_backward.mojo:76-196.
#include "common.cuh"
#include "kernels_api.h"

namespace mdb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}


template <int N>
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&v)[N]) {
  if constexpr (N == 2) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p));
    v[0] = a.x; v[1] = a.y;
  } else if constexpr (N == 4) {
    uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    static_assert(N == 8, "vector width");
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
}
template <int N>
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[N]) {
  if constexpr (N == 2) {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(v[0], v[1]);
  } else if constexpr (N == 4) {
    uint2 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = o;
  } else {
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]);
    o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = o;
  }
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// mode bit 0: 1 = RMSNorm, 0 = LayerNorm
// weight/bias: optional affine [D] (bf16); scale/shift: optional modulation [groups, mod_stride] (bf16)
// out = norm(x) * w + b, then * (1 + scale) + shift
template <int THREADS, int VPT>  // VPT: 8-element vectors per thread (max)
__global__ void __launch_bounds__(THREADS)
norm_modulate_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                         const __nv_bfloat16* __restrict__ weight, const __nv_bfloat16* __restrict__ bias,
                         const __nv_bfloat16* __restrict__ scale, const __nv_bfloat16* __restrict__ shift,
                         float* __restrict__ stats,  // optional [rows,2] (mean, rstd) saved for backward
                         int rows, int D, int ldx, int ldo, int mod_stride, int rows_per_group, float eps, int rms) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nvec = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx);
  float v[VPT][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 u = xr[idx];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = b.x; v[i][3] = b.y;
      v[i][4] = c.x; v[i][5] = c.y; v[i][6] = d.x; v[i][7] = d.y;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s += v[i][j];
        ss += v[i][j] * v[i][j];
      }
    }
  }
  float mean = 0.f, rstd;
  if (rms) {
    ss = block_sum<THREADS>(ss, red);
    rstd = rsqrtf(ss / D + eps);
  } else {
    s = block_sum<THREADS>(s, red);
    mean = s / D;
    // two-pass variance from registers (no cancellation)
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float d = v[i][j] - mean;
          q += d * d;
        }
      }
    }
    q = block_sum<THREADS>(q, red);
    rstd = rsqrtf(q / D + eps);
  }
  if (stats && threadIdx.x == 0) {
    stats[2 * row] = mean;
    stats[2 * row + 1] = rstd;
  }
  const int g = row / rows_per_group;
  const uint4* wv = weight ? reinterpret_cast<const uint4*>(weight) : nullptr;
  const uint4* bv = bias ? reinterpret_cast<const uint4*>(bias) : nullptr;
  const uint4* scv = scale ? reinterpret_cast<const uint4*>(scale + static_cast<size_t>(g) * mod_stride) : nullptr;
  const uint4* shv = shift ? reinterpret_cast<const uint4*>(shift + static_cast<size_t>(g) * mod_stride) : nullptr;
  uint4* orow = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * ldo);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = (v[i][j] - mean) * rstd;
      auto apply = [&](const uint4* p, bool mul, bool plus_one) {
        uint4 u = p[idx];
        uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 f = unpack_bf16x2(w4[k]);
          if (mul) {
            y[2 * k] *= (plus_one ? 1.f + f.x : f.x);
            y[2 * k + 1] *= (plus_one ? 1.f + f.y : f.y);
          } else {
            y[2 * k] += f.x;
            y[2 * k + 1] += f.y;
          }
        }
      };
      if (wv) apply(wv, true, false);
      if (bv) apply(bv, false, false);
      if (scv) apply(scv, true, true);
      if (shv) apply(shv, false, false);
      uint4 o;
      o.x = pack_bf16x2(y[0], y[1]);
      o.y = pack_bf16x2(y[2], y[3]);
      o.z = pack_bf16x2(y[4], y[5]);
      o.w = pack_bf16x2(y[6], y[7]);
      orow[idx] = o;
    }
  }
}

// dx of  y = norm(x) * w (+b) * (1 + scale) (+ shift):   g = dy * w * (1 + scale)
//   LayerNorm: dx = rstd * (g - mean(g) - xhat * mean(g * xhat))
//   RMSNorm  : dx = rstd * (g - xhat * mean(g * xhat))
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
norm_modulate_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                         __nv_bfloat16* __restrict__ dx, const __nv_bfloat16* __restrict__ weight,
                         const __nv_bfloat16* __restrict__ scale, int rows, int D, int ldx, int lddy, int lddx,
                         int mod_stride, int rows_per_group, float eps, int rms) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nvec = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx);
  const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * lddy);
  const int grp = row / rows_per_group;
  const uint4* wv = weight ? reinterpret_cast<const uint4*>(weight) : nullptr;
  const uint4* scv = scale ? reinterpret_cast<const uint4*>(scale + static_cast<size_t>(grp) * mod_stride) : nullptr;
  float v[VPT][8], g[VPT][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 u = xr[idx], w = gr[idx];
      uint32_t a4[4] = {u.x, u.y, u.z, u.w}, g4[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = unpack_bf16x2(a4[k]), h = unpack_bf16x2(g4[k]);
        v[i][2 * k] = f.x; v[i][2 * k + 1] = f.y;
        g[i][2 * k] = h.x; g[i][2 * k + 1] = h.y;
      }
      if (wv) {
        uint4 t = wv[idx];
        uint32_t t4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 f = unpack_bf16x2(t4[k]);
          g[i][2 * k] *= f.x; g[i][2 * k + 1] *= f.y;
        }
      }
      if (scv) {
        uint4 t = scv[idx];
        uint32_t t4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 f = unpack_bf16x2(t4[k]);
          g[i][2 * k] *= 1.f + f.x; g[i][2 * k + 1] *= 1.f + f.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s += v[i][j];
        ss += v[i][j] * v[i][j];
      }
    }
  }
  float mean = 0.f, rstd;
  if (rms) {
    ss = block_sum<THREADS>(ss, red);
    rstd = rsqrtf(ss / D + eps);
  } else {
    s = block_sum<THREADS>(s, red);
    mean = s / D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float d = v[i][j] - mean;
          q += d * d;
        }
      }
    }
    q = block_sum<THREADS>(q, red);
    rstd = rsqrtf(q / D + eps);
  }
  float sg = 0.f, sgx = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float xh = (v[i][j] - mean) * rstd;
        v[i][j] = xh;
        sg += g[i][j];
        sgx += g[i][j] * xh;
      }
    }
  }
  sg = block_sum<THREADS>(sg, red) / D;
  sgx = block_sum<THREADS>(sgx, red) / D;
  if (rms) sg = 0.f;
  uint4* orow = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * lddx);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = rstd * (g[i][j] - sg - v[i][j] * sgx);
      uint4 o;
      o.x = pack_bf16x2(y[0], y[1]);
      o.y = pack_bf16x2(y[2], y[3]);
      o.z = pack_bf16x2(y[4], y[5]);
      o.w = pack_bf16x2(y[6], y[7]);
      orow[idx] = o;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// QK-RMSNorm + RoPE, in place on a packed projection buffer.
//   buf: rows of `row_stride` bf16; a (token, head) vector of Dh elements starts at
//        buf + token*row_stride + part_offset + head*Dh, for part in {q, k}.
//   cos/sin: fp32 [tokens_per_batch, Dh/2] (per token position, shared by heads and batch)
//   One warp per (token, head, part). Dh in {64, 128, 256} (Dh/32 elements per lane, contiguous).
//   interleaved: pairs (2i, 2i+1) use angle i. half-split: pairs (i, i + Dh/2) use angle i.
//   inverse=1 applies the transposed rotation and skips the norm (backward of the rotation).
// ---------------------------------------------------------------------------------------------
template <int DH, int HPW>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(__nv_bfloat16* __restrict__ buf, const __nv_bfloat16* __restrict__ wq,
                    const __nv_bfloat16* __restrict__ wk, const float* __restrict__ cosv,
                    const float* __restrict__ sinv, long long tokens, int tokens_per_batch, int H, int row_stride,
                    int q_off, int k_off, float eps, int interleaved, int inverse, int do_norm, int rope_tokens_start,
                    long long batch_stride, int pos_offset) {
  // One warp owns HPW consecutive heads of one token's q or k: all HPW row loads are issued before any arithmetic
  // (the kernel is latency bound with a single 8-byte load per lane in flight), and the norm weights and the rotary
  // row, which are the same for every head of a token, are read once per warp.
  constexpr int EPL = DH / 32;  // elements per lane
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = H / HPW;
  const long long total = tokens * groups * 2;
  if (warp_global >= total) return;
  const int part = static_cast<int>(warp_global % 2);
  const int head0 = static_cast<int>((warp_global / 2) % groups) * HPW;
  const long long tok = warp_global / (2 * groups);
  const long long bidx = tok / tokens_per_batch;
  const int tin = static_cast<int>(tok % tokens_per_batch);
  __nv_bfloat16* p = buf + bidx * batch_stride + static_cast<long long>(tin) * row_stride + (part ? k_off : q_off) +
                     head0 * DH + lane * EPL;
  const __nv_bfloat16* w = part ? wk : wq;
  const int pos = tin + pos_offset;
  float v[HPW][EPL];
#pragma unroll
  for (int h = 0; h < HPW; ++h) load_vec<EPL>(p + h * DH, v[h]);
  const bool rope = cosv != nullptr && pos >= rope_tokens_start;
  // lane owns elements [lane*EPL, lane*EPL+EPL) for interleaved; for half-split the pair partner (i + DH/2) lives in
  // lane + 16 and comes by shuffle
  const bool upper = lane >= 16;
  float c[EPL], sn[EPL];
  if (rope) {
    const float* cr = cosv + static_cast<size_t>(pos) * (DH / 2);
    const float* sr = sinv + static_cast<size_t>(pos) * (DH / 2);
    const float sgn = inverse ? -1.f : 1.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = lane * EPL + j;
      const int pi = interleaved ? (e >> 1) : (upper ? e - DH / 2 : e);
      if (!interleaved || (j & 1) == 0) {   // an interleaved pair (j, j + 1) shares entry j
        c[j] = cr[pi];
        sn[j] = sr[pi] * sgn;
      } else {
        c[j] = 0.f;
        sn[j] = 0.f;
      }
    }
  }
  float wv[EPL];
  if (do_norm && !inverse) {
    if (w) load_vec<EPL>(w + lane * EPL, wv);
    else {
#pragma unroll
      for (int j = 0; j < EPL; ++j) wv[j] = 1.f;
    }
  }
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    if (do_norm && !inverse) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) ss += v[h][j] * v[h][j];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / DH + eps);
#pragma unroll
      for (int j = 0; j < EPL; ++j)  // round to bf16 after the norm like an unfused bf16 pipeline would
        v[h][j] = __bfloat162float(__float2bfloat16_rn(v[h][j] * r * wv[j]));
    }
    if (rope) {
      if (interleaved) {
#pragma unroll
        for (int j = 0; j < EPL; j += 2) {
          const float a = v[h][j], b = v[h][j + 1];
          v[h][j] = a * c[j] - b * sn[j];
          v[h][j + 1] = a * sn[j] + b * c[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[h][j], 16);
          // lower: a*c - b*s ; upper: b*c + a*s  (a = lower element, b = upper element)
          v[h][j] = upper ? (v[h][j] * c[j] + other * sn[j]) : (v[h][j] * c[j] - other * sn[j]);
        }
      }
    }
    store_vec<EPL>(p + h * DH, v[h]);
  }
}

// Backward of the kernel above, in place on the gradient buffer (same packing as the forward buffer):
// the incoming gradient is rotated back (transposed rotation), then pushed through the RMSNorm using the
// saved raw (pre-norm) projections in xbuf:  dx = rstd * (g*w - xhat * mean(g*w*xhat)).
template <int DH>
__global__ void __launch_bounds__(256)
qk_norm_rope_bwd_kernel(__nv_bfloat16* __restrict__ dbuf, const __nv_bfloat16* __restrict__ xbuf,
                        const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                        const float* __restrict__ cosv, const float* __restrict__ sinv, long long tokens,
                        int tokens_per_batch, int H, int row_stride, int q_off, int k_off, float eps, int interleaved,
                        int do_norm, int rope_tokens_start, long long batch_stride, int pos_offset) {
  constexpr int EPL = DH / 32;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= tokens * H * 2) return;
  const int part = static_cast<int>(warp_global % 2);
  const int head = static_cast<int>((warp_global / 2) % H);
  const long long tok = warp_global / (2 * H);
  const long long bidx = tok / tokens_per_batch;
  const int tin = static_cast<int>(tok % tokens_per_batch);
  const size_t off = bidx * batch_stride + static_cast<long long>(tin) * row_stride + (part ? k_off : q_off) + head * DH;
  const __nv_bfloat16* w = part ? wk : wq;
  const int pos = tin + pos_offset;
  float g[EPL];
  load_vec<EPL>(dbuf + off + lane * EPL, g);
  if (cosv != nullptr && pos >= rope_tokens_start) {
    const float* cr = cosv + static_cast<size_t>(pos) * (DH / 2);
    const float* sr = sinv + static_cast<size_t>(pos) * (DH / 2);
    if (interleaved) {
#pragma unroll
      for (int j = 0; j < EPL; j += 2) {
        const int pi = (lane * EPL + j) >> 1;
        const float c = cr[pi], s = -sr[pi];
        const float a = g[j], b = g[j + 1];
        g[j] = a * c - b * s;
        g[j + 1] = a * s + b * c;
      }
    } else {
      const bool upper = lane >= 16;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, g[j], 16);
        const int e = lane * EPL + j;
        const int pi = upper ? e - DH / 2 : e;
        const float c = cr[pi], s = -sr[pi];
        g[j] = upper ? (g[j] * c + other * s) : (g[j] * c - other * s);
      }
    }
  }
  if (do_norm) {
    float x[EPL];
    load_vec<EPL>(xbuf + off + lane * EPL, x);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) ss += x[j] * x[j];
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / DH + eps);
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float wj = w ? __bfloat162float(w[lane * EPL + j]) : 1.f;
      g[j] *= wj;
      x[j] *= r;
      dot += g[j] * x[j];
    }
    dot = warp_sum(dot) / DH;
#pragma unroll
    for (int j = 0; j < EPL; ++j) g[j] = r * (g[j] - x[j] * dot);
  }
  store_vec<EPL>(dbuf + off + lane * EPL, g);
}

// cos/sin tables from per-token integer-or-float positions on up to 4 axes:
//   angle(t, off_a + i) = pos[t, a] * theta^(-i / half_a),  half_a = axes_dim[a] / 2
__global__ void rope_table_kernel(const float* __restrict__ pos, float* __restrict__ cosv, float* __restrict__ sinv,
                                  int tokens, int naxes, int half_total, int h0, int h1, int h2, int h3, float theta) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * half_total) return;
  const int t = idx / half_total, c = idx % half_total;
  int hs[4] = {h0, h1, h2, h3};
  int a = 0, off = 0;
  while (a < naxes - 1 && c >= off + hs[a]) {
    off += hs[a];
    ++a;
  }
  const int i = c - off;
  // fp64 for the frequency and the range reduction, fp32 sin/cos of the reduced angle
  const double freq = exp(-log(static_cast<double>(theta)) * (static_cast<double>(i) / hs[a]));
  double ang = static_cast<double>(pos[t * naxes + a]) * freq;
  const double two_pi = 6.283185307179586476925286766559;
  ang = ang - floor(ang / two_pi) * two_pi;
  float s, co;
  sincosf(static_cast<float>(ang), &s, &co);
  cosv[idx] = co;
  sinv[idx] = s;
}

}  // namespace mdb

using namespace mdb;

extern "C" int mdb_norm_modulate_fwd(const void* x, void* out, const void* weight, const void* bias, const void* scale,
                                     const void* shift, float* stats, int rows, int D, int ldx, int ldo,
                                     int mod_stride, int rows_per_group, float eps, int rms, cudaStream_t st) {
  if (D % 8 != 0 || D > 16384 || ldx % 8 || ldo % 8 || (scale && mod_stride % 8)) return -1;
  if (rows <= 0) return 0;
  if (rows_per_group <= 0) rows_per_group = rows;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  auto W = reinterpret_cast<const __nv_bfloat16*>(weight);
  auto Bi = reinterpret_cast<const __nv_bfloat16*>(bias);
  auto Sc = reinterpret_cast<const __nv_bfloat16*>(scale);
  auto Sh = reinterpret_cast<const __nv_bfloat16*>(shift);
  const int nvec = D / 8;
  if (nvec <= 128)
    norm_modulate_fwd_kernel<128, 1><<<rows, 128, 0, st>>>(X, O, W, Bi, Sc, Sh, stats, rows, D, ldx, ldo, mod_stride,
                                                            rows_per_group, eps, rms);
  else if (nvec <= 512)
    norm_modulate_fwd_kernel<128, 4><<<rows, 128, 0, st>>>(X, O, W, Bi, Sc, Sh, stats, rows, D, ldx, ldo, mod_stride,
                                                            rows_per_group, eps, rms);
  else
    norm_modulate_fwd_kernel<256, 8><<<rows, 256, 0, st>>>(X, O, W, Bi, Sc, Sh, stats, rows, D, ldx, ldo, mod_stride,
                                                            rows_per_group, eps, rms);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_norm_modulate_bwd(const void* x, const void* dy, void* dx, const void* weight, const void* scale,
                                     int rows, int D, int ldx, int lddy, int lddx, int mod_stride, int rows_per_group,
                                     float eps, int rms, cudaStream_t st) {
  if (D % 8 != 0 || D > 16384 || ldx % 8 || lddy % 8 || lddx % 8 || (scale && mod_stride % 8)) return -1;
  if (rows <= 0) return 0;
  if (rows_per_group <= 0) rows_per_group = rows;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  auto W = reinterpret_cast<const __nv_bfloat16*>(weight);
  auto Sc = reinterpret_cast<const __nv_bfloat16*>(scale);
  const int nvec = D / 8;
  if (nvec <= 128)
    norm_modulate_bwd_kernel<128, 1><<<rows, 128, 0, st>>>(X, DY, DX, W, Sc, rows, D, ldx, lddy, lddx, mod_stride,
                                                            rows_per_group, eps, rms);
  else if (nvec <= 512)
    norm_modulate_bwd_kernel<128, 4><<<rows, 128, 0, st>>>(X, DY, DX, W, Sc, rows, D, ldx, lddy, lddx, mod_stride,
                                                            rows_per_group, eps, rms);
  else
    norm_modulate_bwd_kernel<256, 8><<<rows, 256, 0, st>>>(X, DY, DX, W, Sc, rows, D, ldx, lddy, lddx, mod_stride,
                                                            rows_per_group, eps, rms);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_qk_norm_rope(void* buf, const void* wq, const void* wk, const float* cosv, const float* sinv,
                                long long tokens, int tokens_per_batch, int H, int Dh, int row_stride, int q_off,
                                int k_off, float eps, int interleaved, int inverse, int do_norm, int rope_start,
                                long long batch_stride, int pos_offset, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if ((row_stride % 8) || (q_off % 8) || (k_off % 8) || (batch_stride % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk)) & 15) return -1;   // vector loads of the weights
  const int hpw = (Dh == 256) ? ((H % 2 == 0) ? 2 : 1) : ((H % 4 == 0) ? 4 : (H % 2 == 0) ? 2 : 1);   // heads per warp
  const long long warps = tokens * (H / hpw) * 2;
  const long long blocks = (warps * 32 + 255) / 256;
  auto B = reinterpret_cast<__nv_bfloat16*>(buf);
  auto WQ = reinterpret_cast<const __nv_bfloat16*>(wq);
  auto WK = reinterpret_cast<const __nv_bfloat16*>(wk);
#define MDB_QKNR(DH_, HPW_)                                                                                          \
  qk_norm_rope_kernel<DH_, HPW_><<<static_cast<unsigned>(blocks), 256, 0, st>>>(                                      \
      B, WQ, WK, cosv, sinv, tokens, tokens_per_batch, H, row_stride, q_off, k_off, eps, interleaved, inverse, do_norm, \
      rope_start, batch_stride, pos_offset)
  if (Dh == 128) {
    if (hpw == 4) MDB_QKNR(128, 4); else if (hpw == 2) MDB_QKNR(128, 2); else MDB_QKNR(128, 1);
  } else if (Dh == 64) {
    if (hpw == 4) MDB_QKNR(64, 4); else if (hpw == 2) MDB_QKNR(64, 2); else MDB_QKNR(64, 1);
  } else if (Dh == 256) {
    if (hpw == 2) MDB_QKNR(256, 2); else MDB_QKNR(256, 1);
  } else {
    return -2;
  }
#undef MDB_QKNR
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_qk_norm_rope_bwd(void* dbuf, const void* xbuf, const void* wq, const void* wk, const float* cosv,
                                    const float* sinv, long long tokens, int tokens_per_batch, int H, int Dh,
                                    int row_stride, int q_off, int k_off, float eps, int interleaved, int do_norm,
                                    int rope_start, long long batch_stride, int pos_offset, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if ((row_stride % 8) || (q_off % 8) || (k_off % 8) || (batch_stride % 8)) return -1;
  const long long warps = tokens * H * 2;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  auto D = reinterpret_cast<__nv_bfloat16*>(dbuf);
  auto X = reinterpret_cast<const __nv_bfloat16*>(xbuf);
  auto WQ = reinterpret_cast<const __nv_bfloat16*>(wq);
  auto WK = reinterpret_cast<const __nv_bfloat16*>(wk);
  if (Dh == 128)
    qk_norm_rope_bwd_kernel<128><<<blocks, 256, 0, st>>>(D, X, WQ, WK, cosv, sinv, tokens, tokens_per_batch, H,
                                                         row_stride, q_off, k_off, eps, interleaved, do_norm, rope_start,
        batch_stride, pos_offset);
  else if (Dh == 64)
    qk_norm_rope_bwd_kernel<64><<<blocks, 256, 0, st>>>(D, X, WQ, WK, cosv, sinv, tokens, tokens_per_batch, H,
                                                        row_stride, q_off, k_off, eps, interleaved, do_norm, rope_start,
        batch_stride, pos_offset);
  else if (Dh == 256)
    qk_norm_rope_bwd_kernel<256><<<blocks, 256, 0, st>>>(D, X, WQ, WK, cosv, sinv, tokens, tokens_per_batch, H,
                                                         row_stride, q_off, k_off, eps, interleaved, do_norm, rope_start,
        batch_stride, pos_offset);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_rope_table(const float* pos, float* cosv, float* sinv, int tokens, int naxes, const int* axes_dim,
                              float theta, cudaStream_t st) {
  if (naxes < 1 || naxes > 4) return -1;
  int h[4] = {0, 0, 0, 0};
  int half_total = 0;
  for (int a = 0; a < naxes; ++a) {
    h[a] = axes_dim[a] / 2;
    half_total += h[a];
  }
  const int n = tokens * half_total;
  if (n <= 0) return 0;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, st>>>(pos, cosv, sinv, tokens, naxes, half_total, h[0], h[1], h[2], h[3],
                                                      theta);
  return static_cast<int>(cudaGetLastError());
}
