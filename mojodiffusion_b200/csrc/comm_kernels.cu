// Peer-memory collectives fused with their compute, for one process per GPU over NVLink 5 / NVSwitch.
//
// Every rank maps every peer's buffers (symmetric memory). Kernels read and write peers with plain
// ld/st.global (P2P) or, when an NVLS multicast mapping exists, with multimem.ld_reduce / multimem.st
// (in-switch reduction / broadcast). No TMA multicast is used anywhere.
//
// Synchronisation is by monotonic epoch flags in peer memory: a rank publishes `flags[slot][my_rank] = epoch`
// on every peer with a system-scope release store; waiters poll their own copy with acquire loads and a
// wall-clock bound, after which they record STATUS_TIMEOUT and return (no trap, no endless spin).
//
// Data-parallel LoRA step ("DP all-reduce + grad scale + clip + AdamW" as one fused path):
//   1. dp_reduce_shard   : rank r sums ITS 1/N shard of the flat gradient over all peers (fp32 accumulate), keeps
//                          the fp32 shard locally and accumulates the shard's sum of squares.
//   2. publish_scalar    : the partial sum of squares goes to every peer.
//   3. dp_adamw_shard    : global norm -> clip coefficient -> AdamW on the shard (moments exist only for the
//                          shard: optimizer state is sharded N ways) -> the new bf16 parameters are written to
//                          EVERY rank's parameter buffer (all-gather by direct stores / multimem.st).
// NVLink traffic per rank: (N-1)/N * (grad bytes + param bytes) instead of 2*(N-1)/N * grad bytes for a ring
// all-reduce followed by N redundant optimizer passes over the whole buffer.
//
// The reference has no collective of any kind (serenitymojo/docs/AUDIT_SIMPLETUNER_PARITY_2026-06-11.md:86-110
// describes the missing piece); the AdamW arithmetic matches serenitymojo/training/lora_adamw_plain_fused.mojo.
#include "common.cuh"
#include "comm_api.h"

namespace mdb {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// one thread: publish `value` in flags[slot][rank] of every peer (after making prior writes visible)
__device__ __forceinline__ void signal_all(const MdbPeerTable& flags, int slot, int rank, int world, int value) {
  __threadfence_system();
  for (int r = 0; r < world; ++r) st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * MDB_MAX_RANKS + rank, value);
}

// one thread: wait until every peer's entry in MY flags[slot] reached `value`. Bounded.
__device__ __forceinline__ bool wait_all(const int* my_flags, int slot, int world, int value, int* status, int where) {
  const uint64_t t0 = globaltimer_ns();
  for (int r = 0; r < world; ++r) {
    const int* f = my_flags + slot * MDB_MAX_RANKS + r;
    uint32_t spins = 0;
    while (ld_acquire_sys(f) < value) {
      if ((++spins & 0xffu) == 0 && globaltimer_ns() - t0 > MDB_WAIT_LIMIT_NS) {
        report_status(status, STATUS_TIMEOUT, where, r);
        return false;
      }
    }
  }
  return true;
}

// value > 0: publish / wait for that epoch. value == 0: the epoch is a device-side counter that the kernel itself
// advances (counters[slot] for signals, counters[slots + slot] for waits), so a captured CUDA graph that replays the
// same signal / wait sequence keeps producing fresh epochs without any host-side argument changing.
__global__ void flag_signal_kernel(MdbPeerTable flags, int slot, int rank, int world, int value, int* counters) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (value <= 0) value = ++counters[slot];
    signal_all(flags, slot, rank, world, value);
  }
}
__global__ void flag_wait_kernel(const int* my_flags, int slot, int world, int value, int* counters, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (value <= 0) value = ++counters[MDB_FLAG_SLOTS + slot];
    wait_all(my_flags, slot, world, value, status, 100 + slot);
  }
}

// signal, then wait, in one launch (an all-rank barrier on `slot`); epochs as in the two kernels above
__global__ void flag_barrier_kernel(MdbPeerTable flags, const int* my_flags, int slot, int rank, int world, int value,
                                    int* counters, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int v = value;
    if (v <= 0) { v = ++counters[slot]; counters[MDB_FLAG_SLOTS + slot] = v; }
    signal_all(flags, slot, rank, world, v);
    wait_all(my_flags, slot, world, v, status, 100 + slot);
  }
}

// block-wide: thread 0 waits, everyone learns the outcome
__device__ __forceinline__ bool block_wait_all(const int* my_flags, int slot, int world, int value, int* status,
                                               int where) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = wait_all(my_flags, slot, world, value, status, where) ? 1 : 0;
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void add8_bf16(const uint4& u, float (&acc)[8]) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

// 16 bytes = 8 bf16 summed over all ranks by the switch, fp32 accumulation
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// grads: bf16 flat buffers of `numel` elements on every rank (same offsets). Shard [lo, hi) (multiples of 8).
// red: fp32 [hi - lo] local. sumsq: local fp32 scalar accumulator (zeroed by the caller).
__global__ void __launch_bounds__(256)
dp_reduce_shard_kernel(MdbPeerTable grads, const void* grads_mc, const int* my_flags, int ready_slot, int epoch,
                       int world, long long lo, long long hi, float* __restrict__ red, float* __restrict__ sumsq,
                       int* status) {
  if (!block_wait_all(my_flags, ready_slot, world, epoch, status, 201)) return;
  float acc2 = 0.f;
  const long long nvec = (hi - lo) >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = lo + i * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (grads_mc != nullptr) {
      const uint4 u = multimem_ld_reduce_bf16x8(reinterpret_cast<const __nv_bfloat16*>(grads_mc) + e);
      add8_bf16(u, acc);
    } else {
#pragma unroll 4
      for (int r = 0; r < world; ++r) {
        const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[r]) + e);
        add8_bf16(u, acc);
      }
    }
    float4* o = reinterpret_cast<float4*>(red + i * 8);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc2 += acc[j] * acc[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc2 += __shfl_xor_sync(0xffffffffu, acc2, o);
  __shared__ float s_red[8];
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) s_red[w] = acc2;
  __syncthreads();
  if (w == 0) {
    float t = l < 8 ? s_red[l] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) atomicAdd(sumsq, t);
  }
}

// scalars: symmetric fp32 [MDB_MAX_RANKS] per rank; rank writes its partial into slot `rank` on every peer
// A rank whose status word is not OK (its reduce wait ran out, so *value is incomplete) publishes NaN instead: every
// peer's update kernel then sees a non-finite norm, skips its own update and records the failure on its own device.
__global__ void publish_scalar_kernel(MdbPeerTable scalars, MdbPeerTable flags, const float* value, int slot, int rank,
                                      int world, int epoch, const int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float v = *value;
    if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != STATUS_OK) v = __int_as_float(0x7fc00000);
    for (int r = 0; r < world; ++r) reinterpret_cast<float*>(scalars.p[r])[rank] = v;
    signal_all(flags, slot, rank, world, epoch);
  }
}

struct DpAdam {
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, grad_scale, max_norm;
};

// AdamW on the shard + all-gather of the new parameters. params: bf16 flat buffers on every rank.
// m, v: fp32 [hi - lo] local. done_counter: local int zeroed by the caller; the last block publishes `done_slot`.
__global__ void __launch_bounds__(256)
dp_adamw_shard_kernel(MdbPeerTable params, void* params_mc, MdbPeerTable flags, const int* my_flags,
                      const float* my_scalars, int norm_slot, int done_slot, int epoch, int rank, int world,
                      long long lo, long long hi, const float* __restrict__ red, float* __restrict__ m,
                      float* __restrict__ v, DpAdam h, float* __restrict__ norm_out, int* done_counter, int* status) {
  // A wait that ran out anywhere on this device since the host last read the status word (this kernel's own wait, the
  // reduce kernel before it, a GEMM of the step) means `red` may be stale: skip the update, but still publish the done
  // flag so that the peers' waits end. The host sees the status at its next check and fails the step.
  bool healthy = block_wait_all(my_flags, norm_slot, world, epoch, status, 202);
  healthy = healthy && (status == nullptr || *reinterpret_cast<volatile int*>(status) == STATUS_OK);
  float total = 0.f;
  for (int r = 0; r < world; ++r) total += my_scalars[r];
  if (healthy && !(total == total)) {              // a peer published NaN: its reduce failed
    healthy = false;
    if (threadIdx.x == 0) report_status(status, STATUS_TIMEOUT, 203, 0);
  }
  const float norm = sqrtf(total) * h.grad_scale;
  float clip = 1.f;
  if (h.max_norm > 0.f) {
    const float c = h.max_norm / (norm + 1e-6f);
    clip = c < 1.f ? c : 1.f;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && norm_out != nullptr) *norm_out = norm;
  const float gmul = h.grad_scale * clip;
  const long long nvec = (hi - lo) >> 3;
  __nv_bfloat16* my_params = reinterpret_cast<__nv_bfloat16*>(params.p[rank]);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; healthy && i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = lo + i * 8;
    const uint4 pu = *reinterpret_cast<const uint4*>(my_params + e);
    const uint32_t pw[4] = {pu.x, pu.y, pu.z, pu.w};
    float pf[8], g[8], mm[8], vv[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(pw[k]);
      pf[2 * k] = f.x;
      pf[2 * k + 1] = f.y;
    }
    const float4* gr = reinterpret_cast<const float4*>(red + i * 8);
    const float4 g0 = gr[0], g1 = gr[1];
    g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
    float4* mr = reinterpret_cast<float4*>(m + i * 8);
    float4* vr = reinterpret_cast<float4*>(v + i * 8);
    const float4 m0 = mr[0], m1 = mr[1], v0 = vr[0], v1 = vr[1];
    mm[0] = m0.x; mm[1] = m0.y; mm[2] = m0.z; mm[3] = m0.w; mm[4] = m1.x; mm[5] = m1.y; mm[6] = m1.z; mm[7] = m1.w;
    vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float grad = g[j] * gmul;
      float p = pf[j] * (1.f - h.lr * h.wd);
      mm[j] = h.beta1 * mm[j] + (1.f - h.beta1) * grad;
      vv[j] = h.beta2 * vv[j] + (1.f - h.beta2) * grad * grad;
      p -= (h.lr / h.bc1) * (mm[j] / (sqrtf(vv[j]) / h.bc2_sqrt + h.eps));
      pf[j] = p;
    }
    mr[0] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    mr[1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    vr[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    vr[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 out;
    out.x = pack_bf16x2(pf[0], pf[1]);
    out.y = pack_bf16x2(pf[2], pf[3]);
    out.z = pack_bf16x2(pf[4], pf[5]);
    out.w = pack_bf16x2(pf[6], pf[7]);
    if (params_mc != nullptr) {
      multimem_st_b128(reinterpret_cast<__nv_bfloat16*>(params_mc) + e, out);
    } else {
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + e) = out;
    }
  }
  // last block out publishes "my shard is everywhere"
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(done_counter, 1) == static_cast<int>(gridDim.x) - 1) signal_all(flags, done_slot, rank, world, epoch);
  }
}

// plain all-gather by peer loads: dst = [world chunks]; chunk r comes from src.p[r] (rank r's shard); the local chunk
// is copied too when `copy_local` (otherwise it is expected to be in place already)
__global__ void __launch_bounds__(256)
peer_gather_kernel(MdbPeerTable src, uint4* __restrict__ dst, long long chunk_vec, int rank, int world, int copy_local) {
  for (int i = copy_local ? 0 : 1; i < world; ++i) {
    const int c = (rank + i) % world;
    const uint4* s = reinterpret_cast<const uint4*>(src.p[c]);
    uint4* d = dst + c * chunk_vec;
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < chunk_vec; v += (long long)gridDim.x * blockDim.x)
      d[v] = s[v];
  }
}

static inline int clamp_grid(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = static_cast<long long>(device_sm_count()) * 4;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

// Tail of a staged reduce-scatter: every rank has stored its bf16 partial rows into slot [src] of the row owner's staging
// buffer stage[world][rows][D]. This kernel (1) tells all peers "my partials have landed" (block 0), (2) waits until all
// peers said the same, (3) sums the slots in fp32 and applies bias / gate / residual: out = residual + gate * (sum + bias).
__global__ void __launch_bounds__(256)
rs_finalize_kernel(MdbPeerTable flags, const int* my_flags, int slot, int epoch, int rank, int world,
                   const __nv_bfloat16* __restrict__ stage, long long rows, int D, const __nv_bfloat16* __restrict__ bias,
                   const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ gate, int rows_per_group,
                   long long gate_stride, __nv_bfloat16* __restrict__ out, float* __restrict__ accum, int* status) {
  if (world > 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(flags, slot, rank, world, epoch);
    if (!block_wait_all(my_flags, slot, world, epoch, status, 120 + slot)) return;
  }
  // a wait that ran out earlier in this step (status not yet read by the host): the partial sums may be incomplete, so
  // nothing is written (the peers were signalled above and do not wait for this rank)
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != STATUS_OK) return;
  const long long vec_per_row = D / 8;
  const long long total = rows * vec_per_row;
  const long long slot_elems = rows * static_cast<long long>(D);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / vec_per_row;
    const int col = static_cast<int>(i - row * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s)
      add8_bf16(*reinterpret_cast<const uint4*>(stage + s * slot_elems + row * D + col), acc);
    if (bias) {
      float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8_bf16(*reinterpret_cast<const uint4*>(bias + col), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += b[j];
    }
    if (gate) {
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8_bf16(*reinterpret_cast<const uint4*>(gate + (row / rows_per_group) * gate_stride + col), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= g[j];
    }
    if (residual) add8_bf16(*reinterpret_cast<const uint4*>(residual + row * D + col), acc);
    if (accum) {                                        // gradient accumulation: fp32 shard += reduced partials
      float4* a4 = reinterpret_cast<float4*>(accum + row * D + col);
      float4 lo = a4[0], hi = a4[1];
      lo.x += acc[0]; lo.y += acc[1]; lo.z += acc[2]; lo.w += acc[3];
      hi.x += acc[4]; hi.y += acc[5]; hi.z += acc[6]; hi.w += acc[7];
      a4[0] = lo; a4[1] = hi;
      continue;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + row * D + col) = o;
  }
}

}  // namespace mdb

using namespace mdb;

// Reduce-scatter tail fused with the optimizer (fully-sharded training, one launch per layer inside backward): after the
// same signal / wait as rs_finalize_kernel, every thread adds the N staged bf16 partial gradients of its elements in fp32
// and applies AdamW to the fp32 master shard, its moments, and the bf16 shard the next all-gather reads. The gradient
// shard is never stored. All ranks have finished the input-gradient GEMM that read the OLD shard before they signal, so
// overwriting the bf16 shard here cannot race with a peer's gather of this layer.
struct RsAdam { float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, grad_scale; };
__global__ void __launch_bounds__(256)
rs_adamw_kernel(MdbPeerTable flags, const int* my_flags, int slot, int epoch, int rank, int world,
                const __nv_bfloat16* __restrict__ stage, long long n, float* __restrict__ master, float* __restrict__ m,
                float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, RsAdam h, int* status) {
  if (world > 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(flags, slot, rank, world, epoch);
    if (!block_wait_all(my_flags, slot, world, epoch, status, 140 + slot)) return;
  }
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != STATUS_OK) return;      // see rs_finalize_kernel
  const long long nv = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s) add8_bf16(*reinterpret_cast<const uint4*>(stage + s * n + i * 8), g);
    float4 p0 = *reinterpret_cast<const float4*>(master + i * 8), p1 = *reinterpret_cast<const float4*>(master + i * 8 + 4);
    float4 m0 = *reinterpret_cast<const float4*>(m + i * 8), m1 = *reinterpret_cast<const float4*>(m + i * 8 + 4);
    float4 v0 = *reinterpret_cast<const float4*>(v + i * 8), v1 = *reinterpret_cast<const float4*>(v + i * 8 + 4);
    float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * h.grad_scale;
      pp[j] *= 1.f - h.lr * h.wd;
      mm[j] = h.beta1 * mm[j] + (1.f - h.beta1) * gj;
      vv[j] = h.beta2 * vv[j] + (1.f - h.beta2) * gj * gj;
      pp[j] -= (h.lr / h.bc1) * mm[j] / (sqrtf(vv[j]) / h.bc2_sqrt + h.eps);
    }
    *reinterpret_cast<float4*>(master + i * 8) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    *reinterpret_cast<float4*>(master + i * 8 + 4) = make_float4(pp[4], pp[5], pp[6], pp[7]);
    *reinterpret_cast<float4*>(m + i * 8) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(m + i * 8 + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(v + i * 8) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + i * 8 + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 o;
    o.x = pack_bf16x2(pp[0], pp[1]); o.y = pack_bf16x2(pp[2], pp[3]); o.z = pack_bf16x2(pp[4], pp[5]); o.w = pack_bf16x2(pp[6], pp[7]);
    *reinterpret_cast<uint4*>(shadow + i * 8) = o;
  }
}

extern "C" int mdb_flag_barrier(const MdbPeerTable* flags, const int* my_flags, int slot, int rank, int world, int value,
                                int* counters, int* status, cudaStream_t st) {
  if (slot < 0 || slot >= MDB_FLAG_SLOTS || (value <= 0 && counters == nullptr)) return -1;
  flag_barrier_kernel<<<1, 32, 0, st>>>(*flags, my_flags, slot, rank, world, value, counters, status);
  return (int)cudaGetLastError();
}
extern "C" int mdb_rs_adamw(const MdbPeerTable* flags, const int* my_flags, int slot, int epoch, int rank, int world, const void* stage,
                            long long n, float* master, float* m, float* v, void* shadow, float lr, float beta1, float beta2, float eps,
                            float wd, int step, float grad_scale, int* status, cudaStream_t st) {
  if ((n & 7) || n < 0 || slot < 0 || slot >= MDB_FLAG_SLOTS || epoch <= 0 || step < 1) return -1;
  if (n == 0) return 0;
  RsAdam h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.wd = wd; h.grad_scale = grad_scale;
  h.bc1 = 1.f - powf(beta1, static_cast<float>(step));
  h.bc2_sqrt = sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  const long long want = (n / 8 + 255) / 256;
  const int cap = device_sm_count() * 4;                       // every block waits for the peers: one resident wave
  const int grid = static_cast<int>(want < cap ? want : cap);
  rs_adamw_kernel<<<grid, 256, 0, st>>>(*flags, my_flags, slot, epoch, rank, world, reinterpret_cast<const __nv_bfloat16*>(stage), n, master,
                                        m, v, reinterpret_cast<__nv_bfloat16*>(shadow), h, status);
  return (int)cudaGetLastError();
}
extern "C" int mdb_rs_finalize(const MdbPeerTable* flags, const int* my_flags, int slot, int epoch, int rank, int world,
                               const void* stage, long long rows, int D, const void* bias, const void* residual,
                               const void* gate, int rows_per_group, long long gate_stride, void* out, float* accum,
                               int* status, cudaStream_t st) {
  if (D % 8 || rows < 0 || slot < 0 || slot >= MDB_FLAG_SLOTS || epoch <= 0 || (out == nullptr) == (accum == nullptr)) return -1;
  if (rows == 0) return 0;
  // every block must be resident at once (each waits for the peers): one wave of 4 blocks per SM at most
  const long long want = (rows * (D / 8) + 255) / 256;
  const int cap = device_sm_count() * 4;
  const int grid = static_cast<int>(want < cap ? want : cap);
  rs_finalize_kernel<<<grid, 256, 0, st>>>(*flags, my_flags, slot, epoch, rank, world,
                                           reinterpret_cast<const __nv_bfloat16*>(stage), rows, D,
                                           reinterpret_cast<const __nv_bfloat16*>(bias),
                                           reinterpret_cast<const __nv_bfloat16*>(residual),
                                           reinterpret_cast<const __nv_bfloat16*>(gate), rows_per_group > 0 ? rows_per_group : 1,
                                           gate_stride, reinterpret_cast<__nv_bfloat16*>(out), accum, status);
  return (int)cudaGetLastError();
}

extern "C" int mdb_flag_signal(const MdbPeerTable* flags, int slot, int rank, int world, int value, int* counters,
                               cudaStream_t st) {
  if (slot < 0 || slot >= MDB_FLAG_SLOTS || (value <= 0 && counters == nullptr)) return -1;
  flag_signal_kernel<<<1, 32, 0, st>>>(*flags, slot, rank, world, value, counters);
  return (int)cudaGetLastError();
}
extern "C" int mdb_flag_wait(const int* my_flags, int slot, int world, int value, int* counters, int* status,
                             cudaStream_t st) {
  if (slot < 0 || slot >= MDB_FLAG_SLOTS || (value <= 0 && counters == nullptr)) return -1;
  flag_wait_kernel<<<1, 32, 0, st>>>(my_flags, slot, world, value, counters, status);
  return (int)cudaGetLastError();
}
extern "C" int mdb_peer_gather(const MdbPeerTable* src, void* dst, long long chunk_bytes, int rank, int world,
                               int copy_local, cudaStream_t st) {
  if (chunk_bytes & 15) return -1;
  if (chunk_bytes == 0) return 0;
  peer_gather_kernel<<<clamp_grid(chunk_bytes / 16, 256), 256, 0, st>>>(*src, reinterpret_cast<uint4*>(dst),
                                                                        chunk_bytes / 16, rank, world, copy_local);
  return (int)cudaGetLastError();
}
extern "C" int mdb_dp_reduce_shard(const MdbPeerTable* grads, const void* grads_mc, const int* my_flags, int ready_slot,
                                   int epoch, int world, long long lo, long long hi, float* red, float* sumsq,
                                   int* status, cudaStream_t st) {
  if ((lo & 7) || (hi & 7) || hi < lo) return -1;
  if (hi == lo) return 0;
  dp_reduce_shard_kernel<<<clamp_grid((hi - lo) / 8, 256), 256, 0, st>>>(*grads, grads_mc, my_flags, ready_slot, epoch,
                                                                        world, lo, hi, red, sumsq, status);
  return (int)cudaGetLastError();
}
extern "C" int mdb_publish_scalar(const MdbPeerTable* scalars, const MdbPeerTable* flags, const float* value, int slot,
                                  int rank, int world, int epoch, const int* status, cudaStream_t st) {
  publish_scalar_kernel<<<1, 32, 0, st>>>(*scalars, *flags, value, slot, rank, world, epoch, status);
  return (int)cudaGetLastError();
}
extern "C" int mdb_dp_adamw_shard(const MdbPeerTable* params, void* params_mc, const MdbPeerTable* flags,
                                  const int* my_flags, const float* my_scalars, int norm_slot, int done_slot, int epoch,
                                  int rank, int world, long long lo, long long hi, const float* red, float* m, float* v,
                                  float lr, float beta1, float beta2, float eps, float wd, int step, float grad_scale,
                                  float max_norm, float* norm_out, int* done_counter, int* status, cudaStream_t st) {
  if ((lo & 7) || (hi & 7) || hi < lo) return -1;
  DpAdam h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.wd = wd;
  h.bc1 = 1.f - powf(beta1, (float)step);
  h.bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  h.grad_scale = grad_scale; h.max_norm = max_norm;
  const int grid = hi > lo ? clamp_grid((hi - lo) / 8, 256) : 1;
  dp_adamw_shard_kernel<<<grid, 256, 0, st>>>(*params, params_mc, *flags, my_flags, my_scalars, norm_slot, done_slot,
                                              epoch, rank, world, lo, hi, red, m, v, h, norm_out, done_counter, status);
  return (int)cudaGetLastError();
}

MDB_DEFINE_WAIT_LIMIT_SETTER(mdb_set_wait_limit_comm)
