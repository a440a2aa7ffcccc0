// Attention backward for sm_100a on tcgen05 / TMEM. Two launches of one templated kernel:
//
//   KV_MODE = false (dQ):    CTA owns 128 query rows, streams 64-key tiles:
//        X = Q K_j^T, Y = dO V_j^T  ->  dS = P o (Y - delta)  ->  dQ += dS K_j
//   KV_MODE = true  (dK,dV): CTA owns 128 key rows, streams 64-query tiles:
//        X = K Q_i^T, Y = V dO_i^T  ->  P^T, dS^T             ->  dV += P^T dO_i ; dK += dS^T Q_i
//
// with P = exp(scale * S - lse) rebuilt from the forward's log-sum-exp and delta = rowsum(dO o O), so no
// [S, S] tensor ever exists in memory. The 128-row operands (R tiles) stay in shared memory for the whole CTA,
// the 64-row operands (C tiles) stream through a 3-stage TMA ring and serve twice: K-major as the B operand of
// the score GEMMs and MN-major as the B operand of the gradient GEMMs (same bytes, different descriptor).
// Score tiles X, Y are double buffered in TMEM so the tensor core computes tile i+1 while the math warps turn
// tile i into bf16 P / dS, which they write back into TMEM over X / Y as the A operand (TS-form) of the
// gradient GEMMs. TMEM: X0 X1 Y0 Y1 (64 columns each) + two 128-column accumulators = 512 columns.
//
// Math matched: serenitymojo/ops/attention_backward.mojo:249-349 (7-step decomposed backward) and the cuDNN
// flash backward the reference binds (serenitymojo/ops/cshim/cudnn_sdpa_bwd.cpp:325).
#include "common.cuh"
#include <stdlib.h>
#include "gemm_api.h"
#include "kernels_api.h"

#include <string.h>

namespace mdb {

constexpr int BWD_THREADS = 192;
constexpr int RB = 128;  // resident rows per CTA
constexpr int CB = 64;   // streamed rows per tile
constexpr int CST = 3;   // C ring stages

struct alignas(64) BwdMaps {
  CUtensorMap r1, r2, c1, c2;
};

struct BwdParams {
  __nv_bfloat16* out1;  // dQ (dQ mode) or dK (KV mode)
  __nv_bfloat16* out2;  // dV (KV mode)
  long long o1_strides[3], o2_strides[3];  // (batch, seq, head)
  const float* lse;     // [B, H, Sq] natural log
  const float* delta;   // [B, H, Sq]
  const int* kv_len;
  int B, H, Sq, Skv;
  float scale, scale_log2;
  int exp_poly;
  int* status;
};

// delta[b, h, q] = sum_d dO[b,q,h,d] * O[b,q,h,d]; one warp per (b, q, h) row
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int B, int Sq, int H, int Dh, long long os0,
                                  long long os1, long long os2, long long ds0, long long ds1, long long ds2) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * Sq * H) return;
  const int h = static_cast<int>(w % H);
  const int q = static_cast<int>((w / H) % Sq);
  const int b = static_cast<int>(w / ((long long)H * Sq));
  const __nv_bfloat16* po = o + b * os0 + q * os1 + h * os2;
  const __nv_bfloat16* pd = dout + b * ds0 + q * ds1 + h * ds2;
  float acc = 0.f;
  for (int c = lane * 2; c < Dh; c += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(po + c));
    float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + c));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[((long long)b * H + h) * Sq + q] = acc;
}

template <int DH, bool KV_MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ BwdMaps maps, const BwdParams p) {
  constexpr int DBOX = DH / 64;
  constexpr int R_BYTES = RB * DH * 2;       // one resident tile
  constexpr int R_BOX = RB * 128;            // 128 rows x 128 B
  constexpr int C_BYTES = CB * DH * 2;       // one streamed tile
  constexpr int C_BOX = CB * 128;            // 64 rows x 128 B
  constexpr uint32_t X_COL = 0, Y_COL = 128, ACC1_COL = 256, ACC2_COL = 384;  // X0 X1 | Y0 Y1 | acc1 | acc2

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t r_full, c_full[CST], c_empty[CST], xy_full[2], pds_full[2], lv_full[2], acc_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ __align__(8) float s_lse2[2][CB], s_delta[2][CB];      // NEGATED lse * log2(e) and delta per staged query

  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sR1 = smem;
  uint8_t* sR2 = sR1 + R_BYTES;
  uint8_t* sC = sR2 + R_BYTES;  // CST stages of (C1, C2)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int r0 = blockIdx.x * RB;

  int kv_valid = p.Skv;
  if (p.kv_len != nullptr) kv_valid = min(kv_valid, p.kv_len[batch]);
  if (kv_valid < 1) kv_valid = 1;
  const int c_extent = KV_MODE ? p.Sq : kv_valid;  // rows of the streamed dimension that matter
  const int n_c = (c_extent + CB - 1) / CB;
  const int out_rows = KV_MODE ? p.Skv : p.Sq;

  if (KV_MODE && r0 >= kv_valid) {
    // keys that no query attends to: zero gradients, nothing to compute
    for (int idx = threadIdx.x; idx < RB * (DH / 8); idx += BWD_THREADS) {
      const int row = r0 + idx / (DH / 8), c = (idx % (DH / 8)) * 8;
      if (row < out_rows) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(p.out1 + batch * p.o1_strides[0] + (long long)row * p.o1_strides[1] +
                                  head * p.o1_strides[2] + c) = z;
        *reinterpret_cast<uint4*>(p.out2 + batch * p.o2_strides[0] + (long long)row * p.o2_strides[1] +
                                  head * p.o2_strides[2] + c) = z;
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&r_full, 1);
    for (int s = 0; s < CST; ++s) {
      mbar_init(&c_full[s], 1);
      mbar_init(&c_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&xy_full[s], 1);
      mbar_init(&pds_full[s], 128);
      mbar_init(&lv_full[s], CB);
    }
    mbar_init(&acc_full, 1);
    abort_s = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&maps.r1);
    tma_prefetch_desc(&maps.r2);
    tma_prefetch_desc(&maps.c1);
    tma_prefetch_desc(&maps.c2);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      // ----------------------------- TMA producer -----------------------------
      mbar_expect_tx(&r_full, 2 * R_BYTES);
      for (int d = 0; d < DBOX; ++d) {
        tma_load_4d(sR1 + d * R_BOX, &maps.r1, &r_full, d * 64, r0, head, batch);
        tma_load_4d(sR2 + d * R_BOX, &maps.r2, &r_full, d * 64, r0, head, batch);
      }
      bool ok = true;
      uint64_t* last_bar = &r_full;
      uint32_t last_par = 0;
      int st = 0;
      uint32_t par = 0;
      for (int i = 0; ok && i < n_c; ++i) {
        if (!mbar_wait(&c_empty[st], par ^ 1u, &abort_s)) {
          report_status(p.status, STATUS_TIMEOUT, 41, i);
          ok = false;
          break;
        }
        uint8_t* c1 = sC + st * 2 * C_BYTES;
        uint8_t* c2 = c1 + C_BYTES;
        mbar_expect_tx(&c_full[st], 2 * C_BYTES);
        for (int d = 0; d < DBOX; ++d) {
          tma_load_4d(c1 + d * C_BOX, &maps.c1, &c_full[st], d * 64, i * CB, head, batch);
          tma_load_4d(c2 + d * C_BOX, &maps.c2, &c_full[st], d * 64, i * CB, head, batch);
        }
        last_bar = &c_full[st];
        last_par = par;
        if (++st == CST) {
          st = 0;
          par ^= 1u;
        }
      }
      if (!ok) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(last_bar, last_par) && globaltimer_ns() - t0 < 5000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ----------------------------- UMMA issuer ------------------------------
      constexpr uint32_t idesc_xy = make_idesc(1, UMMA_BF16, UMMA_BF16, 0, 0, RB, CB);
      constexpr uint32_t idesc_acc = make_idesc(1, UMMA_BF16, UMMA_BF16, 0, 1, RB, DH);
      auto issue_xy = [&](int st, int buf) {
        const uint32_t a1 = smem_u32(sR1), a2 = smem_u32(sR2);
        const uint32_t b1 = smem_u32(sC + st * 2 * C_BYTES), b2 = b1 + C_BYTES;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t offa = (kk / 4) * R_BOX + (kk % 4) * 32;
          const uint32_t offb = (kk / 4) * C_BOX + (kk % 4) * 32;
          umma_f16_ss(tmem_base + X_COL + buf * CB, make_desc_kmajor_sw128(a1 + offa),
                      make_desc_kmajor_sw128(b1 + offb), idesc_xy, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t offa = (kk / 4) * R_BOX + (kk % 4) * 32;
          const uint32_t offb = (kk / 4) * C_BOX + (kk % 4) * 32;
          umma_f16_ss(tmem_base + Y_COL + buf * CB, make_desc_kmajor_sw128(a2 + offa),
                      make_desc_kmajor_sw128(b2 + offb), idesc_xy, kk != 0 ? 1u : 0u);
        }
        umma_commit(&xy_full[buf]);
      };
      auto issue_acc = [&](int st, int buf, bool first) {
        const uint32_t b1 = smem_u32(sC + st * 2 * C_BYTES), b2 = b1 + C_BYTES;
        // acc1 += dS (over Y) * C1 ; KV mode: acc2 += P^T (over X) * C2
#pragma unroll
        for (int kk = 0; kk < CB / 16; ++kk)
          umma_f16_ts(tmem_base + ACC1_COL, tmem_base + Y_COL + buf * CB + kk * 8,
                      make_desc_mnmajor_sw128(b1 + kk * 2048, C_BOX), idesc_acc, (first && kk == 0) ? 0u : 1u);
        if (KV_MODE) {
#pragma unroll
          for (int kk = 0; kk < CB / 16; ++kk)
            umma_f16_ts(tmem_base + ACC2_COL, tmem_base + X_COL + buf * CB + kk * 8,
                        make_desc_mnmajor_sw128(b2 + kk * 2048, C_BOX), idesc_acc, (first && kk == 0) ? 0u : 1u);
        }
      };
      bool ok = mbar_wait(&r_full, 0, &abort_s) && mbar_wait(&c_full[0], 0, &abort_s);
      if (!ok) report_status(p.status, STATUS_TIMEOUT, 51, 0);
      if (ok) {
        tc_fence_after();
        issue_xy(0, 0);
      }
      for (int i = 0; ok && i < n_c; ++i) {
        const int st = i % CST;
        if (i + 1 < n_c) {
          const int stn = (i + 1) % CST;
          if (!mbar_wait(&c_full[stn], ((i + 1) / CST) & 1, &abort_s)) {
            report_status(p.status, STATUS_TIMEOUT, 52, i);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_xy(stn, (i + 1) & 1);
        }
        if (!mbar_wait(&pds_full[i & 1], (i >> 1) & 1, &abort_s)) {
          report_status(p.status, STATUS_TIMEOUT, 53, i);
          ok = false;
          break;
        }
        tc_fence_after();
        issue_acc(st, i & 1, i == 0);
        umma_commit(&c_empty[st]);
      }
      if (ok) umma_commit(&acc_full);
    }
    __syncwarp();
  } else {
    // ------------------------------- math warps (128 threads) --------------------------
    const int quad = warp & 3;
    const int mt = quad * 32 + lane;  // row inside the resident tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int row = r0 + mt;
    const long long lse_base = (static_cast<long long>(batch) * p.H + head) * p.Sq;
    const float LOG2E = 1.4426950408889634f;
    float my_lse2 = INFINITY, my_delta = 0.f;
    if (!KV_MODE && row < p.Sq) {
      my_lse2 = p.lse[lse_base + row] * LOG2E;
      my_delta = p.delta[lse_base + row];
    }
    const bool row_key_valid = KV_MODE ? (row < kv_valid) : true;
    bool ok = true;
    for (int i = 0; i < n_c; ++i) {
      const int buf = i & 1;
      if (KV_MODE) {
        // per-query lse / delta of this 64-query tile, staged by the first 64 math threads. The buffer was last
        // read in iteration i-2: its 128 readers have all arrived on pds_full[buf] for that iteration.
        bool lv_ok = true;
        if (mt < CB) {
          if (i >= 2) lv_ok = mbar_wait(&pds_full[buf], ((i - 2) >> 1) & 1, &abort_s);
          const int q = i * CB + mt;
          s_lse2[buf][mt] = q < p.Sq ? -p.lse[lse_base + q] * LOG2E : -INFINITY;
          s_delta[buf][mt] = q < p.Sq ? -p.delta[lse_base + q] : 0.f;
          mbar_arrive(&lv_full[buf]);
        }
        lv_ok = mbar_wait(&lv_full[buf], (i >> 1) & 1, &abort_s) && lv_ok;
        if (!__all_sync(0xffffffffu, lv_ok)) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 60, i);
          ok = false;
          break;
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(&xy_full[buf], (i >> 1) & 1, &abort_s));
      if (!ok) {
        if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 61, i);
        break;
      }
      tc_fence_after();
      const uint32_t xa = tmem_base + lane_addr + X_COL + buf * CB;
      const uint32_t ya = tmem_base + lane_addr + Y_COL + buf * CB;
#pragma unroll
      for (int c = 0; c < CB / 32; ++c) {
        uint32_t xr[32], yr[32];
        tmem_ld_32x32b_x32(xa + c * 32, xr);
        tmem_ld_32x32b_x32(ya + c * 32, yr);
        tmem_wait_ld();
        uint32_t pk[16], dk[16];
        // Four columns per step as packed pairs: exponent = x * scale - lse2 and (dP - delta) are one packed operation
        // each; with exp_poly the odd columns' exponentials run as a packed polynomial on the FMA pipe.
        const float2 sl2_2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 my_nl2 = make_float2(-my_lse2, -my_lse2), my_ndl = make_float2(-my_delta, -my_delta);
        const bool tail = !KV_MODE && (i * CB + CB > kv_valid);
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const int col = c * 32 + e;
          float2 nl01, nl23, nd01, nd23;
          if (KV_MODE) {
            nl01 = *reinterpret_cast<const float2*>(&s_lse2[buf][col]);
            nl23 = *reinterpret_cast<const float2*>(&s_lse2[buf][col + 2]);
            nd01 = *reinterpret_cast<const float2*>(&s_delta[buf][col]);
            nd23 = *reinterpret_cast<const float2*>(&s_delta[buf][col + 2]);
          } else {
            nl01 = nl23 = my_nl2;
            nd01 = nd23 = my_ndl;
          }
          const float2 x01 = ffma2(make_float2(__uint_as_float(xr[e]), __uint_as_float(xr[e + 1])), sl2_2, nl01);
          const float2 x23 = ffma2(make_float2(__uint_as_float(xr[e + 2]), __uint_as_float(xr[e + 3])), sl2_2, nl23);
          float2 p01, p23;
          if (p.exp_poly) {
            const float2 b = ex2_poly2(make_float2(x01.y, x23.y));
            p01 = make_float2(ex2_approx(x01.x), b.x);
            p23 = make_float2(ex2_approx(x23.x), b.y);
          } else {
            p01 = make_float2(ex2_approx(x01.x), ex2_approx(x01.y));
            p23 = make_float2(ex2_approx(x23.x), ex2_approx(x23.y));
          }
          if (KV_MODE) {
            if (!row_key_valid) p01 = p23 = make_float2(0.f, 0.f);
          } else if (tail) {
            const int k0 = i * CB + col;
            if (k0 >= kv_valid) p01.x = 0.f;
            if (k0 + 1 >= kv_valid) p01.y = 0.f;
            if (k0 + 2 >= kv_valid) p23.x = 0.f;
            if (k0 + 3 >= kv_valid) p23.y = 0.f;
          }
          const float2 d01 = fmul2(p01, fadd2(make_float2(__uint_as_float(yr[e]), __uint_as_float(yr[e + 1])), nd01));
          const float2 d23 = fmul2(p23, fadd2(make_float2(__uint_as_float(yr[e + 2]), __uint_as_float(yr[e + 3])), nd23));
          pk[e >> 1] = pack_bf16x2(p01.x, p01.y);
          pk[(e >> 1) + 1] = pack_bf16x2(p23.x, p23.y);
          dk[e >> 1] = pack_bf16x2(d01.x, d01.y);
          dk[(e >> 1) + 1] = pack_bf16x2(d23.x, d23.y);
        }
        if (KV_MODE) tmem_st_32x32b_x16(xa + c * 16, pk);
        tmem_st_32x32b_x16(ya + c * 16, dk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&pds_full[buf]);
    }
    if (ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full, 0, &abort_s));
      if (!ok && lane == 0) report_status(p.status, STATUS_TIMEOUT, 62, 0);
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* o1 = p.out1 + batch * p.o1_strides[0] + static_cast<long long>(row) * p.o1_strides[1] +
                          head * p.o1_strides[2];
      __nv_bfloat16* o2 = KV_MODE ? p.out2 + batch * p.o2_strides[0] + static_cast<long long>(row) * p.o2_strides[1] +
                                        head * p.o2_strides[2]
                                  : nullptr;
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + ACC1_COL + c * 32, r);
        tmem_wait_ld();
        if (row < out_rows) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[e + 0]) * p.scale, __uint_as_float(r[e + 1]) * p.scale);
            w.y = pack_bf16x2(__uint_as_float(r[e + 2]) * p.scale, __uint_as_float(r[e + 3]) * p.scale);
            w.z = pack_bf16x2(__uint_as_float(r[e + 4]) * p.scale, __uint_as_float(r[e + 5]) * p.scale);
            w.w = pack_bf16x2(__uint_as_float(r[e + 6]) * p.scale, __uint_as_float(r[e + 7]) * p.scale);
            *reinterpret_cast<uint4*>(o1 + c * 32 + e) = w;
          }
        }
        if (KV_MODE) {
          tmem_ld_32x32b_x32(tmem_base + lane_addr + ACC2_COL + c * 32, r);
          tmem_wait_ld();
          if (row < out_rows) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(r[e + 0]), __uint_as_float(r[e + 1]));
              w.y = pack_bf16x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
              w.z = pack_bf16x2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
              w.w = pack_bf16x2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
              *reinterpret_cast<uint4*>(o2 + c * 32 + e) = w;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DH, bool KV_MODE>
static int launch_bwd(const BwdMaps& maps, const BwdParams& p, int rows, cudaStream_t st) {
  constexpr int SMEM = 2 * RB * DH * 2 + CST * 2 * CB * DH * 2 + 1024;
  auto kern = attention_bwd_kernel<DH, KV_MODE>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  dim3 grid((rows + RB - 1) / RB, p.H, p.B);
  kern<<<grid, BWD_THREADS, SMEM, st>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

static int make_map(CUtensorMap* m, const void* ptr, int B, int S, int H, int Dh, const long long* strides,
                    int box_rows) {
  int64_t ext[4] = {Dh, S, H, B};
  int64_t str[4] = {2, strides[1] * 2, strides[2] * 2, strides[0] * 2};
  int box[4] = {64, box_rows, 1, 1};
  return mdb_make_tmap(m, ptr, 2, 4, ext, str, box, 1);
}

}  // namespace mdb

extern "C" int mdb_attention_bwd(const MdbAttnBwdArgs* a, cudaStream_t st) {
  using namespace mdb;
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Skv <= 0) return -1;
  if (a->Dh != 128 && a->Dh != 64) return -2;
  for (int i = 0; i < 3; ++i) {
    if ((a->q_strides[i] % 8) || (a->k_strides[i] % 8) || (a->v_strides[i] % 8) || (a->o_strides[i] % 8) ||
        (a->do_strides[i] % 8) || (a->dq_strides[i] % 8) || (a->dk_strides[i] % 8) || (a->dv_strides[i] % 8))
      return -3;
  }
  // delta = rowsum(dO o O)
  {
    const long long rows = static_cast<long long>(a->B) * a->Sq * a->H;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    attn_delta_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(a->o),
                                              reinterpret_cast<const __nv_bfloat16*>(a->dout), a->delta, a->B, a->Sq,
                                              a->H, a->Dh, a->o_strides[0], a->o_strides[1], a->o_strides[2],
                                              a->do_strides[0], a->do_strides[1], a->do_strides[2]);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  BwdParams p;
  memset(&p, 0, sizeof(p));
  p.lse = a->lse;
  p.delta = a->delta;
  p.kv_len = a->kv_len;
  p.B = a->B; p.H = a->H; p.Sq = a->Sq; p.Skv = a->Skv;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  {
    static int mode = -1;
    if (mode < 0) {
      const char* e = getenv("MDB200_ATTN_EXP_POLY");
      mode = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    p.exp_poly = mode;
  }
  p.status = a->status;
  int r;
  // ---- dQ: resident Q, dO ; streamed K, V
  {
    BwdMaps maps;
    if ((r = make_map(&maps.r1, a->q, a->B, a->Sq, a->H, a->Dh, a->q_strides, RB))) return 1000 + r;
    if ((r = make_map(&maps.r2, a->dout, a->B, a->Sq, a->H, a->Dh, a->do_strides, RB))) return 1100 + r;
    if ((r = make_map(&maps.c1, a->k, a->B, a->Skv, a->H, a->Dh, a->k_strides, CB))) return 1200 + r;
    if ((r = make_map(&maps.c2, a->v, a->B, a->Skv, a->H, a->Dh, a->v_strides, CB))) return 1300 + r;
    p.out1 = reinterpret_cast<__nv_bfloat16*>(a->dq);
    p.out2 = nullptr;
    for (int i = 0; i < 3; ++i) p.o1_strides[i] = a->dq_strides[i];
    r = a->Dh == 128 ? launch_bwd<128, false>(maps, p, a->Sq, st) : launch_bwd<64, false>(maps, p, a->Sq, st);
    if (r) return r;
  }
  // ---- dK, dV: resident K, V ; streamed Q, dO
  {
    BwdMaps maps;
    if ((r = make_map(&maps.r1, a->k, a->B, a->Skv, a->H, a->Dh, a->k_strides, RB))) return 2000 + r;
    if ((r = make_map(&maps.r2, a->v, a->B, a->Skv, a->H, a->Dh, a->v_strides, RB))) return 2100 + r;
    if ((r = make_map(&maps.c1, a->q, a->B, a->Sq, a->H, a->Dh, a->q_strides, CB))) return 2200 + r;
    if ((r = make_map(&maps.c2, a->dout, a->B, a->Sq, a->H, a->Dh, a->do_strides, CB))) return 2300 + r;
    p.out1 = reinterpret_cast<__nv_bfloat16*>(a->dk);
    p.out2 = reinterpret_cast<__nv_bfloat16*>(a->dv);
    for (int i = 0; i < 3; ++i) {
      p.o1_strides[i] = a->dk_strides[i];
      p.o2_strides[i] = a->dv_strides[i];
    }
    r = a->Dh == 128 ? launch_bwd<128, true>(maps, p, a->Skv, st) : launch_bwd<64, true>(maps, p, a->Skv, st);
    if (r) return r;
  }
  return 0;
}

MDB_DEFINE_WAIT_LIMIT_SETTER(mdb_set_wait_limit_attn_bwd)
