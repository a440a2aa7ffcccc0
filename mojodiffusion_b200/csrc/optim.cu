// Fused optimizer kernels for sm_100a: multi-tensor AdamW in ONE launch (fp32 or bf16 params, fp32 or
// bf16 gradients, fp32 or bf16 moments, optional stochastic-rounding bf16 write-back and an optional bf16
// shadow copy of fp32 masters), on-device global gradient norm, and the clip coefficient taken from
// that norm on the device so no host sync sits between backward and the update.
//
// Update order is torch.optim.AdamW's: p *= 1 - lr*wd; m,v EMA; p -= lr/bc1 * m / (sqrt(v)/sqrt(bc2) + eps).
// Reference behaviour matched: serenitymojo/training/optim.mojo:79-338, serenitymojo/training/fused_adamw_multitensor.mojo:45-285,
// serenitymojo/training/lora_adamw_ot_fused.mojo:75-142 (bf16 moments + stochastic rounding),
// serenitymojo/training/lora_adamw_plain_fused.mojo, serenitymojo/training/on_device_global_norm.mojo:1-169,
// serenitymojo/util/bf16_stochastic_rounding.mojo:13-73.
#include "common.cuh"
#include "kernels_api.h"

namespace mdb {

__device__ __forceinline__ uint32_t hash_u32(uint32_t a, uint32_t b, uint32_t c) {
  // 3-word mix (murmur-style finaliser rounds); good enough for rounding dither
  uint32_t h = a * 0x9E3779B1u ^ (b + 0x7F4A7C15u) * 0x85EBCA77u ^ (c + 0x165667B1u) * 0xC2B2AE3Du;
  h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
  return h;
}
// stochastic rounding fp32 -> bf16: add 16 uniform random bits below the kept mantissa, truncate
__device__ __forceinline__ __nv_bfloat16 sr_bf16(float x, uint32_t rnd) {
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return __float2bfloat16_rn(x);  // inf / nan unchanged
  u += (rnd & 0xffffu);
  __nv_bfloat16_raw r;
  r.x = static_cast<unsigned short>(u >> 16);
  return __nv_bfloat16(r);
}

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

struct AdamHyper {
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt;  // bc1 = 1 - beta1^t ; bc2_sqrt = sqrt(1 - beta2^t)
  float grad_scale;                                 // static multiplier on every gradient (1/world, 1/accum)
  const float* norm_sq;                             // optional device scalar: sum of squares of the scaled grads
  float max_norm;                                   // clip threshold (<=0: off)
  unsigned int seed;                                // stochastic rounding stream
  int stochastic;                                   // bf16 params only
  const int* status;                                // optional device status word: not OK (a bounded wait of this step
                                                    // ran out, gradients may be incomplete) -> nothing is updated
};

__device__ __forceinline__ float clip_coef(const AdamHyper& h) {
  if (h.norm_sq == nullptr || h.max_norm <= 0.f) return 1.f;
  const float norm = sqrtf(*h.norm_sq) * h.grad_scale;
  const float c = h.max_norm / (norm + 1e-6f);
  return c < 1.f ? c : 1.f;
}

template <typename TP, typename TG, typename TM>
__device__ __forceinline__ void adamw_elem(TP* p, const TG* g, TM* m, TM* v, __nv_bfloat16* shadow, long long i,
                                           const AdamHyper& h, float gmul, uint32_t tensor_id) {
  const float grad = ldf<TG>(g, i) * gmul;
  float pv = ldf<TP>(p, i);
  float mv = ldf<TM>(m, i);
  float vv = ldf<TM>(v, i);
  pv *= (1.f - h.lr * h.wd);
  mv = h.beta1 * mv + (1.f - h.beta1) * grad;
  vv = h.beta2 * vv + (1.f - h.beta2) * grad * grad;
  const float denom = sqrtf(vv) / h.bc2_sqrt + h.eps;
  pv -= (h.lr / h.bc1) * (mv / denom);
  stf<TM>(m, i, mv);
  stf<TM>(v, i, vv);
  if constexpr (sizeof(TP) == 2) {
    if (h.stochastic)
      p[i] = sr_bf16(pv, hash_u32(h.seed, tensor_id, static_cast<uint32_t>(i)));
    else
      p[i] = __float2bfloat16_rn(pv);
  } else {
    p[i] = pv;
    if (shadow) shadow[i] = __float2bfloat16_rn(pv);
  }
}

// chunk table: each entry = (tensor index, first element); a block walks chunks grid-stride
template <typename TP, typename TG, typename TM>
__global__ void __launch_bounds__(256)
adamw_multi_kernel(const MdbTensorEntry* __restrict__ tensors, const int2* __restrict__ chunks, int num_chunks,
                   int chunk_elems, AdamHyper h) {
  if (h.status != nullptr && *reinterpret_cast<const volatile int*>(h.status) != STATUS_OK) return;
  const float gmul = h.grad_scale * clip_coef(h);
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ch = chunks[c];
    const MdbTensorEntry t = tensors[ch.x];
    const long long start = static_cast<long long>(ch.y) * chunk_elems;
    const long long end = min(start + static_cast<long long>(chunk_elems), t.numel);
    TP* p = reinterpret_cast<TP*>(t.param);
    const TG* g = reinterpret_cast<const TG*>(t.grad);
    TM* m = reinterpret_cast<TM*>(t.exp_avg);
    TM* v = reinterpret_cast<TM*>(t.exp_avg_sq);
    __nv_bfloat16* sh = reinterpret_cast<__nv_bfloat16*>(t.shadow);
    for (long long i = start + threadIdx.x; i < end; i += blockDim.x)
      adamw_elem<TP, TG, TM>(p, g, m, v, sh, i, h, gmul, static_cast<uint32_t>(ch.x));
  }
}

template <typename TG>
__global__ void __launch_bounds__(256)
sumsq_multi_kernel(const MdbTensorEntry* __restrict__ tensors, const int2* __restrict__ chunks, int num_chunks,
                   int chunk_elems, float* __restrict__ out) {
  float acc = 0.f;
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ch = chunks[c];
    const MdbTensorEntry t = tensors[ch.x];
    const long long start = static_cast<long long>(ch.y) * chunk_elems;
    const long long end = min(start + static_cast<long long>(chunk_elems), t.numel);
    const TG* g = reinterpret_cast<const TG*>(t.grad);
    for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
      const float x = ldf<TG>(g, i);
      acc += x * x;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float red[8];
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = acc;
  __syncthreads();
  if (w == 0) {
    float t = l < 8 ? red[l] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) atomicAdd(out, t);
  }
}

// p_ema = decay * p_ema + (1 - decay) * p   (fp32 ema, any param dtype) over a chunk table
template <typename TP>
__global__ void __launch_bounds__(256)
ema_multi_kernel(const MdbTensorEntry* __restrict__ tensors, const int2* __restrict__ chunks, int num_chunks,
                 int chunk_elems, float decay) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ch = chunks[c];
    const MdbTensorEntry t = tensors[ch.x];
    const long long start = static_cast<long long>(ch.y) * chunk_elems;
    const long long end = min(start + static_cast<long long>(chunk_elems), t.numel);
    const TP* p = reinterpret_cast<const TP*>(t.param);
    float* e = reinterpret_cast<float*>(t.exp_avg);
    for (long long i = start + threadIdx.x; i < end; i += blockDim.x)
      e[i] = decay * e[i] + (1.f - decay) * ldf<TP>(p, i);
  }
}

}  // namespace mdb

using namespace mdb;
typedef __nv_bfloat16 bf16;

extern "C" int mdb_adamw_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems,
                               int p_bf16, int g_bf16, int m_bf16, float lr, float beta1, float beta2, float eps,
                               float wd, int step, float grad_scale, const float* norm_sq, float max_norm,
                               unsigned int seed, int stochastic, const int* status, cudaStream_t st) {
  if (num_chunks <= 0) return 0;
  AdamHyper h;
  h.status = status;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.wd = wd;
  h.bc1 = 1.f - powf(beta1, (float)step);
  h.bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  h.grad_scale = grad_scale; h.norm_sq = norm_sq; h.max_norm = max_norm; h.seed = seed; h.stochastic = stochastic;
  const int cap = device_sm_count() * 8;
  const int grid = num_chunks < cap ? num_chunks : cap;
  const int2* ch = reinterpret_cast<const int2*>(chunks);
#define MDB_AD(TP, TG, TM) adamw_multi_kernel<TP, TG, TM><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, h)
  if (p_bf16) {
    if (g_bf16) { if (m_bf16) MDB_AD(bf16, bf16, bf16); else MDB_AD(bf16, bf16, float); }
    else        { if (m_bf16) MDB_AD(bf16, float, bf16); else MDB_AD(bf16, float, float); }
  } else {
    if (g_bf16) { if (m_bf16) MDB_AD(float, bf16, bf16); else MDB_AD(float, bf16, float); }
    else        { if (m_bf16) MDB_AD(float, float, bf16); else MDB_AD(float, float, float); }
  }
#undef MDB_AD
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Lion and StableAdamW over the same tensor table (fp32 moments; fp32 or bf16 parameters and gradients)
// ---------------------------------------------------------------------------------------------
// Lion: update = sign(beta1 m + (1 - beta1) g); p = p (1 - lr wd) - lr update; m = beta2 m + (1 - beta2) g
template <typename TP, typename TG>
__global__ void __launch_bounds__(256)
lion_multi_kernel(const MdbTensorEntry* __restrict__ tensors, const int2* __restrict__ chunks, int num_chunks,
                  int chunk_elems, float lr, float beta1, float beta2, float wd, float gmul, const int* status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != STATUS_OK) return;
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ch = chunks[c];
    const MdbTensorEntry t = tensors[ch.x];
    const long long start = static_cast<long long>(ch.y) * chunk_elems;
    const long long end = min(start + static_cast<long long>(chunk_elems), t.numel);
    TP* p = reinterpret_cast<TP*>(t.param);
    const TG* g = reinterpret_cast<const TG*>(t.grad);
    float* m = reinterpret_cast<float*>(t.exp_avg);
    for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
      const float grad = ldf<TG>(g, i) * gmul;
      const float mv = m[i];
      const float cdir = beta1 * mv + (1.f - beta1) * grad;
      const float upd = cdir > 0.f ? 1.f : (cdir < 0.f ? -1.f : 0.f);
      stf<TP>(p, i, ldf<TP>(p, i) * (1.f - lr * wd) - lr * upd);
      m[i] = beta2 * mv + (1.f - beta2) * grad;
    }
  }
}

// StableAdamW, pass 1: moments with the debiased betas, and per tensor the sum of g^2 / max(v, eps^2)
template <typename TG>
__global__ void __launch_bounds__(256)
stable_adamw_moments_kernel(const MdbTensorEntry* __restrict__ tensors, const int2* __restrict__ chunks, int num_chunks,
                            int chunk_elems, float beta1h, float beta2h, float eps, float gmul,
                            float* __restrict__ rms_acc, const int* status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != STATUS_OK) return;
  __shared__ float red[8];
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ch = chunks[c];
    const MdbTensorEntry t = tensors[ch.x];
    const long long start = static_cast<long long>(ch.y) * chunk_elems;
    const long long end = min(start + static_cast<long long>(chunk_elems), t.numel);
    const TG* g = reinterpret_cast<const TG*>(t.grad);
    float* m = reinterpret_cast<float*>(t.exp_avg);
    float* v = reinterpret_cast<float*>(t.exp_avg_sq);
    float acc = 0.f;
    for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
      const float grad = ldf<TG>(g, i) * gmul;
      m[i] = beta1h * m[i] + (1.f - beta1h) * grad;
      const float vv = beta2h * v[i] + (1.f - beta2h) * grad * grad;
      v[i] = vv;
      acc += grad * grad / fmaxf(vv, eps * eps);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = acc;
    __syncthreads();
    if (w == 0) {
      float s = l < 8 ? red[l] : 0.f;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (l == 0) atomicAdd(rms_acc + ch.x, s);
    }
    __syncthreads();
  }
}

// StableAdamW, pass 2: eta = lr / max(1, sqrt(rms_acc / numel)); p = p (1 - eta wd) - eta m / (sqrt(v) + eps)
template <typename TP>
__global__ void __launch_bounds__(256)
stable_adamw_update_kernel(const MdbTensorEntry* __restrict__ tensors, const int2* __restrict__ chunks, int num_chunks,
                           int chunk_elems, float lr, float eps, float wd, const float* __restrict__ rms_acc,
                           const int* status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != STATUS_OK) return;
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ch = chunks[c];
    const MdbTensorEntry t = tensors[ch.x];
    const long long start = static_cast<long long>(ch.y) * chunk_elems;
    const long long end = min(start + static_cast<long long>(chunk_elems), t.numel);
    TP* p = reinterpret_cast<TP*>(t.param);
    const float* m = reinterpret_cast<const float*>(t.exp_avg);
    const float* v = reinterpret_cast<const float*>(t.exp_avg_sq);
    const float rms = sqrtf(rms_acc[ch.x] / static_cast<float>(t.numel));
    const float eta = lr / fmaxf(1.f, rms);
    for (long long i = start + threadIdx.x; i < end; i += blockDim.x)
      stf<TP>(p, i, ldf<TP>(p, i) * (1.f - eta * wd) - eta * m[i] / (sqrtf(v[i]) + eps));
  }
}

extern "C" int mdb_lion_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems, int p_bf16,
                              int g_bf16, float lr, float beta1, float beta2, float wd, float grad_scale,
                              const int* status, cudaStream_t st) {
  if (num_chunks <= 0) return 0;
  const int cap = device_sm_count() * 8;
  const int grid = num_chunks < cap ? num_chunks : cap;
  const int2* ch = reinterpret_cast<const int2*>(chunks);
#define MDB_LION(TP, TG) lion_multi_kernel<TP, TG><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, lr, beta1, beta2, wd, grad_scale, status)
  if (p_bf16) { if (g_bf16) MDB_LION(bf16, bf16); else MDB_LION(bf16, float); }
  else        { if (g_bf16) MDB_LION(float, bf16); else MDB_LION(float, float); }
#undef MDB_LION
  return (int)cudaGetLastError();
}

// rms_acc: one zeroed float per tensor of the table
extern "C" int mdb_stable_adamw_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems,
                                      int p_bf16, int g_bf16, float lr, float beta1h, float beta2h, float eps, float wd,
                                      float grad_scale, float* rms_acc, const int* status, cudaStream_t st) {
  if (num_chunks <= 0) return 0;
  const int cap = device_sm_count() * 8;
  const int grid = num_chunks < cap ? num_chunks : cap;
  const int2* ch = reinterpret_cast<const int2*>(chunks);
  if (g_bf16) stable_adamw_moments_kernel<bf16><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, beta1h, beta2h, eps, grad_scale, rms_acc, status);
  else stable_adamw_moments_kernel<float><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, beta1h, beta2h, eps, grad_scale, rms_acc, status);
  if (p_bf16) stable_adamw_update_kernel<bf16><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, lr, eps, wd, rms_acc, status);
  else stable_adamw_update_kernel<float><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, lr, eps, wd, rms_acc, status);
  return (int)cudaGetLastError();
}

extern "C" int mdb_sumsq_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems,
                               int g_bf16, float* out, cudaStream_t st) {
  if (num_chunks <= 0) return 0;
  const int cap = device_sm_count() * 8;
  const int grid = num_chunks < cap ? num_chunks : cap;
  const int2* ch = reinterpret_cast<const int2*>(chunks);
  if (g_bf16)
    sumsq_multi_kernel<bf16><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, out);
  else
    sumsq_multi_kernel<float><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, out);
  return (int)cudaGetLastError();
}

extern "C" int mdb_ema_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems,
                             int p_bf16, float decay, cudaStream_t st) {
  if (num_chunks <= 0) return 0;
  const int cap = device_sm_count() * 8;
  const int grid = num_chunks < cap ? num_chunks : cap;
  const int2* ch = reinterpret_cast<const int2*>(chunks);
  if (p_bf16)
    ema_multi_kernel<bf16><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, decay);
  else
    ema_multi_kernel<float><<<grid, 256, 0, st>>>(tensors, ch, num_chunks, chunk_elems, decay);
  return (int)cudaGetLastError();
}


// ---------------------------------------------------------------------------------
// AdamW with 8-bit block-wise quantised moments: each block of 256 elements stores its two moments as indices into a
// 256-entry non-uniform code book (signed for the first moment, unsigned for the second) plus one fp32 absolute maximum
// per block and moment. One CTA = one block: de-quantise through the code books staged in shared memory, update, write
// the parameter, find the new block maxima, re-quantise to the nearest code (binary search, ties to the smaller code).
// Role of the reference's serenitymojo/training/adamw8bit.mojo (32 KB of fp32 optimizer state per million parameters
// instead of 8 MB).
// ---------------------------------------------------------------------------------
namespace mdb {
__device__ __forceinline__ int nearest_code(const float* code, float x) {
  // smallest idx with code[idx] >= x, clamped to [1, 255]  (matches a left bisection)
  int lo = 0, hi = 256;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int mid = (lo + hi) >> 1;
    if (code[mid] < x) lo = mid + 1; else hi = mid;
  }
  int idx = lo < 1 ? 1 : (lo > 255 ? 255 : lo);
  const float a = code[idx - 1], b = code[idx];
  return (fabsf(x - a) <= fabsf(b - x)) ? idx - 1 : idx;
}

template <typename PT, typename GT>
__global__ void __launch_bounds__(256) adamw8bit_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                        uint8_t* __restrict__ qm, uint8_t* __restrict__ qv,
                                                        float* __restrict__ am, float* __restrict__ av,
                                                        const float* __restrict__ code_s, const float* __restrict__ code_u,
                                                        long long n, float lr, float b1, float b2, float eps, float wd,
                                                        float bc1, float bc2_sqrt, float grad_scale, int first) {
  __shared__ float cs[256], cu[256];
  __shared__ float red_m[8], red_v[8];
  cs[threadIdx.x] = code_s[threadIdx.x];
  cu[threadIdx.x] = code_u[threadIdx.x];
  __syncthreads();
  for (long long blk = blockIdx.x; blk * 256 < n; blk += gridDim.x) {
    const long long i = blk * 256 + threadIdx.x;
    const bool in = i < n;
    float m = 0.f, v = 0.f, gv = 0.f;
    if (in) {
      gv = static_cast<float>(g[i]) * grad_scale;
      if (!first) {
        m = cs[qm[i]] * am[blk];
        v = cu[qv[i]] * av[blk];
      }
      m = b1 * m + (1.f - b1) * gv;
      v = b2 * v + (1.f - b2) * gv * gv;
      float pf = static_cast<float>(p[i]) * (1.f - lr * wd);
      pf -= (lr / bc1) * m / (sqrtf(v) / bc2_sqrt + eps);
      p[i] = static_cast<PT>(pf);
    }
    float mx = in ? fabsf(m) : 0.f, vx = in ? fabsf(v) : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      vx = fmaxf(vx, __shfl_xor_sync(0xffffffffu, vx, o));
    }
    if ((threadIdx.x & 31) == 0) {
      red_m[threadIdx.x >> 5] = mx;
      red_v[threadIdx.x >> 5] = vx;
    }
    __syncthreads();
    mx = red_m[0];
    vx = red_v[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      mx = fmaxf(mx, red_m[w]);
      vx = fmaxf(vx, red_v[w]);
    }
    mx = fmaxf(mx, 1e-30f);
    vx = fmaxf(vx, 1e-30f);
    if (in) {
      qm[i] = static_cast<uint8_t>(nearest_code(cs, m / mx));
      qv[i] = static_cast<uint8_t>(nearest_code(cu, v / vx));
    }
    if (threadIdx.x == 0) {
      am[blk] = mx;
      av[blk] = vx;
    }
    __syncthreads();
  }
}
}  // namespace mdb

extern "C" int mdb_adamw8bit(void* p, const void* g, void* qm, void* qv, float* am, float* av, const float* code_s,
                             const float* code_u, long long n, int p_bf16, int g_bf16, float lr, float b1, float b2, float eps,
                             float wd, int step, float grad_scale, cudaStream_t st) {
  using namespace mdb;
  if (n <= 0) return 0;
  const long long blocks = (n + 255) / 256;
  const long long cap16 = static_cast<long long>(device_sm_count()) * 16;
  const int grid = static_cast<int>(blocks < cap16 ? blocks : cap16);
  const float bc1 = 1.f - powf(b1, static_cast<float>(step));
  const float bc2s = sqrtf(1.f - powf(b2, static_cast<float>(step)));
  const int first = step <= 1;
  uint8_t* a = static_cast<uint8_t*>(qm);
  uint8_t* b = static_cast<uint8_t*>(qv);
#define MDB_A8(PT, GT)                                                                                               \
  adamw8bit_kernel<PT, GT><<<grid, 256, 0, st>>>(static_cast<PT*>(p), static_cast<const GT*>(g), a, b, am, av, code_s, \
                                                 code_u, n, lr, b1, b2, eps, wd, bc1, bc2s, grad_scale, first)
  if (p_bf16 && g_bf16) MDB_A8(__nv_bfloat16, __nv_bfloat16);
  else if (p_bf16) MDB_A8(__nv_bfloat16, float);
  else if (g_bf16) MDB_A8(float, __nv_bfloat16);
  else MDB_A8(float, float);
#undef MDB_A8
  return static_cast<int>(cudaGetLastError());
}
