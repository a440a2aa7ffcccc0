// Block-scaled fp8 GEMM on the 5th-generation tensor cores: out[M, N] (bf16) = A[M, K] * B[N, K]^T with both operands in
// the MXFP8 format (E4M3 elements, one E8M0 scale 2^(b - 127) per 32 consecutive K elements of a row), scales applied by
// the hardware inside tcgen05.mma kind::mxf8f6f4.block_scale. Replaces the reference's weight-only fp8 kernel with a
// 16 x 16 shared-memory tile (serenitymojo/ops/fp8_gemm.mojo:28-73) and its fp8 quantisers (serenitymojo/ops/fp8_quant.mojo).
//
//   * One CTA per 128 x 256 output tile, 192 threads: warp 0 feeds a 4-stage ring by TMA (A 128 x 128 B, B 256 x 128 B,
//     128-byte swizzle, plus the scale chunks by untiled bulk copies), warp 1 issues, warps 2-5 drain the accumulator.
//   * Scales travel in the layout the tensor core reads: per 128 rows and 4 scale columns (= 128 K elements) one 512-byte
//     chunk, byte (row % 32) * 16 + (row / 32) * 4 + column. A chunk is copied to 4 TMEM columns by one
//     tcgen05.cp 32x128b.warpx4; the scale id fields of the instruction descriptor select the byte for each K = 32 MMA.
//     (Measured on the device with one-hot scale patterns: every row / column / id picks exactly this byte.)
//   * Rows past M / N are zero-filled by TMA; their scale chunks exist (buffers are padded to whole tiles and preset to
//     127 = 1.0, because the byte 255 is NaN in E8M0 and NaN * 0 would poison the sum).
//   * Every wait is bounded: on expiry the CTA sets its abort flag, records STATUS_TIMEOUT and leaves through the common
//     exit, where its TMEM is freed.
#include "common.cuh"
#include "kernels_api.h"
#include <cuda_fp8.h>
#include <algorithm>

namespace mdb {

constexpr int MX_BM = 128, MX_BN = 256, MX_BK = 128;          // K block in fp8 elements = bytes
constexpr int MX_STAGES = 4;
constexpr int MX_A_BYTES = MX_BM * MX_BK, MX_B_BYTES = MX_BN * MX_BK;
constexpr int MX_SF_CHUNK = 512;
constexpr int MX_STAGE_BYTES = MX_A_BYTES + MX_B_BYTES + 3 * MX_SF_CHUNK;
constexpr int MX_SMEM = MX_STAGES * MX_STAGE_BYTES + 1024;
constexpr int MX_THREADS = 192;
constexpr uint32_t MX_SF_COL0 = 256, MX_SF_COLS_PER_STAGE = 16;  // accumulator in columns 0..255

struct MxMaps { CUtensorMap a, b; };
struct MxParams {
  const uint8_t* sfa;        // [ceil(M/128)][K/128][512]
  const uint8_t* sfb;        // [2 * ceil(N/256)][K/128][512]
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  int M, N, K, ld_out;
  int* status;
};

__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                             uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// block-scaled instruction descriptor: [4,6) B scale id, [7,10) A format, [10,13) B format (0 = E4M3), [17,23) N >> 3,
// [23] scale format (1 = E8M0), [24,29) M >> 4, [29,31) A scale id
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t M, uint32_t N, uint32_t sf_id) {
  return (sf_id << 4) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (sf_id << 29);
}

__global__ void __launch_bounds__(MX_THREADS, 1) gemm_mxfp8_kernel(const __grid_constant__ MxMaps maps, const MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[MX_STAGES], empty_bar[MX_STAGES], acc_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * MX_BN, m0 = blockIdx.y * MX_BM;
  const int kblocks = p.K / MX_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MX_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_bar, 1);
    abort_s = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&maps.a); tma_prefetch_desc(&maps.b); }
  if (warp == 1) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ---------------------------------- producer ----------------------------------
    const uint8_t* sfa = p.sfa + static_cast<size_t>(blockIdx.y) * kblocks * MX_SF_CHUNK;
    const uint8_t* sfb0 = p.sfb + static_cast<size_t>(2 * blockIdx.x) * kblocks * MX_SF_CHUNK;
    const uint8_t* sfb1 = sfb0 + static_cast<size_t>(kblocks) * MX_SF_CHUNK;
    bool ok = true;
    for (int kb = 0; ok && kb < kblocks; ++kb) {
      const int st = kb % MX_STAGES;
      const uint32_t par = ((kb / MX_STAGES) & 1) ^ 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[st], par, &abort_s));
      if (!ok) { if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 301, kb); break; }
      if (elect_one()) {
        uint8_t* sA = smem + st * MX_STAGE_BYTES;
        uint8_t* sB = sA + MX_A_BYTES;
        uint8_t* sS = sB + MX_B_BYTES;
        mbar_expect_tx(&full_bar[st], MX_A_BYTES + MX_B_BYTES + 3 * MX_SF_CHUNK);
        tma_load_2d(sA, &maps.a, &full_bar[st], kb * MX_BK, m0);
        tma_load_2d(sB, &maps.b, &full_bar[st], kb * MX_BK, n0);
        tma_load_2d(sB + MX_B_BYTES / 2, &maps.b, &full_bar[st], kb * MX_BK, n0 + 128);
        bulk_load_g2s(sS, sfa + static_cast<size_t>(kb) * MX_SF_CHUNK, MX_SF_CHUNK, &full_bar[st]);
        bulk_load_g2s(sS + MX_SF_CHUNK, sfb0 + static_cast<size_t>(kb) * MX_SF_CHUNK, MX_SF_CHUNK, &full_bar[st]);
        bulk_load_g2s(sS + 2 * MX_SF_CHUNK, sfb1 + static_cast<size_t>(kb) * MX_SF_CHUNK, MX_SF_CHUNK, &full_bar[st]);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------------------------- MMA issuer ----------------------------------
    bool ok = true;
    for (int kb = 0; ok && kb < kblocks; ++kb) {
      const int st = kb % MX_STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[st], (kb / MX_STAGES) & 1, &abort_s));
      if (!ok) { if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 302, kb); break; }
      tc_fence_after();
      if (elect_one()) {
        const uint32_t sA = smem_u32(smem + st * MX_STAGE_BYTES);
        const uint32_t sB = sA + MX_A_BYTES, sS = sB + MX_B_BYTES;
        const uint32_t sf = tmem_base + MX_SF_COL0 + st * MX_SF_COLS_PER_STAGE;
        // scale chunks: [32 rows][16 bytes] contiguous = four 8-row core matrices 128 bytes apart, no swizzle
        tmem_cp_32x128b_warpx4(sf, make_smem_desc(sS, 128, 128, 0));
        tmem_cp_32x128b_warpx4(sf + 4, make_smem_desc(sS + MX_SF_CHUNK, 128, 128, 0));
        tmem_cp_32x128b_warpx4(sf + 8, make_smem_desc(sS + 2 * MX_SF_CHUNK, 128, 128, 0));
        const uint64_t da = make_desc_kmajor_sw128(sA), db = make_desc_kmajor_sw128(sB);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_mxf8_ss(tmem_base, da + ((k * 32) >> 4), db + ((k * 32) >> 4), make_idesc_mx(MX_BM, MX_BN, k), sf, sf + 4,
                       (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[st]);
        if (kb == kblocks - 1) umma_commit(&acc_bar);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------- epilogue ----------------------------------
    const int quad = warp & 3;                              // TMEM lane quadrant this warp may read
    const int row = m0 + quad * 32 + lane;
    bool ok = __all_sync(0xffffffffu, mbar_wait(&acc_bar, 0, &abort_s));
    if (!ok && lane == 0) report_status(p.status, STATUS_TIMEOUT, 303, 0);
    if (ok) {
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < MX_BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row < p.M) {
          __nv_bfloat16* o = p.out + static_cast<size_t>(row) * p.ld_out + col0;
          if (col0 + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[i + j]) + (p.bias ? __bfloat162float(p.bias[col0 + i + j]) : 0.f);
              uint4 w;
              w.x = pack_bf16x2(v[0], v[1]); w.y = pack_bf16x2(v[2], v[3]); w.z = pack_bf16x2(v[4], v[5]); w.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(o + i) = w;
            }
          } else {
            for (int i = 0; i < 32 && col0 + i < p.N; ++i)
              o[i] = __float2bfloat16_rn(__uint_as_float(r[i]) + (p.bias ? __bfloat162float(p.bias[col0 + i]) : 0.f));
          }
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---- quantiser: bf16 rows -> E4M3 bytes + scale chunks in the tensor core's layout -------------------------------------
__device__ __forceinline__ float mx_pow2i(int e) { return __uint_as_float(static_cast<uint32_t>(e + 127) << 23); }
__device__ __forceinline__ float mx_mul_exact(float a, float b) { float d; asm("mul.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }

// one thread per (row, 32-element block)
__global__ void mxfp8_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                        long long rows, int K, long long ldx) {
  const int kb32 = K / 32;
  const long long total = rows * kb32;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / kb32;
    const int kb = static_cast<int>(t - r * kb32);
    const uint4* in = reinterpret_cast<const uint4*>(x + r * ldx + kb * 32);
    float v[32];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = in[i];
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[i * 8 + 0] = a.x; v[i * 8 + 1] = a.y; v[i * 8 + 2] = b.x; v[i * 8 + 3] = b.y;
      v[i * 8 + 4] = c.x; v[i * 8 + 5] = c.y; v[i * 8 + 6] = d.x; v[i * 8 + 7] = d.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    int eb = 0;
    if (amax > 0.f) eb = min(max(static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 8, 0), 254);
    const int ie = 127 - eb;
    const float ia = mx_pow2i(ie / 2), ib = mx_pow2i(ie - ie / 2);
    uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 32; ++i)
      w[i >> 2] |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(mx_mul_exact(mx_mul_exact(v[i], ia), ib), __NV_SATFINITE, __NV_E4M3)) << ((i & 3) * 8);
    uint4* out = reinterpret_cast<uint4*>(q + r * K + kb * 32);
    out[0] = make_uint4(w[0], w[1], w[2], w[3]);
    out[1] = make_uint4(w[4], w[5], w[6], w[7]);
    const long long chunk = (r / 128) * (K / 128) + kb / 4;
    const int rin = static_cast<int>(r % 128);
    sf[chunk * 512 + (rin % 32) * 16 + (rin / 32) * 4 + (kb % 4)] = static_cast<uint8_t>(eb);
  }
}

}  // namespace mdb

extern "C" int mdb_make_tmap(void* out_map, const void* ptr, int elem_bytes, int rank, const int64_t* extents,
                             const int64_t* strides_bytes, const int* box, int swizzle128);

extern "C" int mdb_mxfp8_quant_rows(const void* x, void* q, void* sf, long long rows, int K, long long ldx, cudaStream_t st) {
  if (K % 128 || ldx % 8) return -1;
  if (rows == 0) return 0;
  const long long total = rows * (K / 32);
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148 * 16));
  mdb::mxfp8_quant_rows_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q),
                                                        reinterpret_cast<uint8_t*>(sf), rows, K, ldx);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mdb_gemm_mxfp8(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* out, const void* bias, int M,
                              int N, int K, int ld_out, int* status, cudaStream_t st) {
  using namespace mdb;
  if (M <= 0 || N <= 0) return 0;
  if (K % MX_BK || N % 8 || ld_out % 8) return -1;
  MxMaps maps;
  const int64_t ext_a[2] = {K, M}, ext_b[2] = {K, N}, str[2] = {1, K};
  const int box[2] = {MX_BK, 128};
  int r = mdb_make_tmap(&maps.a, a_q, 1, 2, ext_a, str, box, 1);
  if (r) return r;
  r = mdb_make_tmap(&maps.b, b_q, 1, 2, ext_b, str, box, 1);
  if (r) return r;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  MxParams p;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K; p.ld_out = ld_out; p.status = status;
  dim3 grid((N + MX_BN - 1) / MX_BN, (M + MX_BM - 1) / MX_BM);
  gemm_mxfp8_kernel<<<grid, MX_THREADS, MX_SMEM, st>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

MDB_DEFINE_WAIT_LIMIT_SETTER(mdb_set_wait_limit_mxfp8)
