// Flash-style attention forward for sm_100a on the 5th-generation tensor cores.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles that take turns: while all eight
// softmax warps work on one tile's S, the tensor core runs the other tile's P*V and next Q*K^T.
//   * Q (2 x 128 x Dh), K and V (128 x Dh, double buffered) arrive by TMA straight from the caller's
//     [batch, seq, head, Dh] strides (4-D tensor maps, 128-byte swizzle): no head transpose pass exists.
//   * S = Q K^T  : tcgen05.mma SS-form, fp32 accumulator in TMEM (128 columns per tile).
//   * softmax    : two threads per query row (64 key columns each, no shuffles; the row maximum is exchanged through
//                  shared memory), exp2 with the scale folded in, P written back into TMEM as packed bf16 over the S
//                  columns it came from. A per-kv-tile time line (mdb_attention_set_trace) showed the kernel bound by the
//                  softmax chain, not by the tensor core; one thread per row with one warpgroup per tile measured the
//                  same throughput with twice the registers.
//   * O += P V   : tcgen05.mma TS-form (A = P from TMEM, B = V MN-major from shared memory) accumulating in a
//                  second TMEM region across all key tiles. The running maximum used for the exponent is only
//                  raised when a row's true maximum exceeds it by more than 2^8 ("lazy rescale"): then, and
//                  only then, the warp scales its rows of O in TMEM. P stays below 256, exact in fp32 sums.
//   * 512 TMEM columns: S0 S1 O0 O1.
// Keys beyond Skv or beyond kv_len[b] are masked; ragged Sq / Skv tiles are zero filled by TMA.
//
// Takes the place of the reference's math-mode SDPA (serenitymojo/ops/attention.mojo:68-520), its scalar
// online-softmax kernels (:734-873,1109-1167) and its cuDNN flash shim (serenitymojo/ops/cshim/cudnn_sdpa.cpp:375,470;
// Stats/LSE output as in the training forward there).
#include "common.cuh"
#include <stdlib.h>
#include "gemm_api.h"
#include "kernels_api.h"

#include <string.h>

namespace mdb {

constexpr int ATT_THREADS = 384;  // warps 0-3: control warpgroup (TMA, UMMA issue, 2 idle); 4-11: two softmax warpgroups
#ifndef MDB_ATT_CTRL_REGS
#define MDB_ATT_CTRL_REGS 88
#define MDB_ATT_SOFTMAX_REGS 208
#endif
constexpr int CTRL_REGS = MDB_ATT_CTRL_REGS, SOFTMAX_REGS = MDB_ATT_SOFTMAX_REGS;  // 128*ctrl + 256*softmax <= 384*168
constexpr int BQ = 128;   // rows per q tile
constexpr int BKV = 128;  // keys per kv tile

#ifndef MDB_ATTN_ISSUE_DEFAULT
#define MDB_ATTN_ISSUE_DEFAULT 1
#endif
#ifndef MDB_ATTN_POLY_DEFAULT
#define MDB_ATTN_POLY_DEFAULT 2
#endif
static long long* g_attn_trace = nullptr;
static int g_attn_trace_len = 0;

struct alignas(64) AttnMaps {
  CUtensorMap q, k, v;
};

struct AttnParams {
  __nv_bfloat16* o;
  float* lse;
  const int* kv_len;
  int B, H, Sq, Skv;
  long long o_strides[3];
  float scale_log2;
  int exp_poly;   // MDB200_ATTN_EXP_POLY=N (1, 2, 4): one exponential in 2N runs as a polynomial on the FMA pipe; 0: none.
                  // Measured at S=4608, H=24: 0.374 ms (0), 0.374 (1), 0.361 (2, the default), 0.419 (4).
  int* status;
  void* o_route_a[8];
  void* o_route_b[8];
  int route_rows_a, route_split, route_rows_b;
  long long* trace;   // optional time line of CTA (0,0,0): [4 roles][trace_len] clock64 values (see mdb_attention_set_trace)
  int trace_len;
};

template <int REGS> __device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS> __device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}

// How the two control warps run their loops. MODE 0: one lane runs the whole role inside a branch. MODE 1: the whole warp
// runs the loop, every lane polls the barriers, elect.sync picks the issuing lane. MODE 2: the whole warp runs the loop,
// lane 0 polls and broadcasts the outcome, elect.sync picks the issuing lane (a convergent warp issues TMA / tcgen05
// instructions cheaper, and one polling lane keeps the traffic on barriers the softmax warps arrive on low).
template <int MODE> __device__ __forceinline__ bool ctl_wait(uint64_t* bar, uint32_t par, int* abort_flag, int lane) {
  if (MODE == 0) return mbar_wait(bar, par, abort_flag);
  if (MODE == 1) return __all_sync(0xffffffffu, mbar_wait(bar, par, abort_flag));
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, par, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
template <int MODE> __device__ __forceinline__ bool ctl_issuer() { return MODE == 0 ? true : elect_one() != 0; }
template <int MODE> __device__ __forceinline__ void ctl_rejoin() {
  if (MODE != 0) __syncwarp();
}

template <int DH, int MODE, int POLY_EVERY>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ AttnMaps maps, const AttnParams p) {
  constexpr int DBOX = DH / 64;               // 64-element (128 B) boxes along the head dim
  constexpr int TILE_BYTES = BQ * DH * 2;     // one 128-row operand tile
  constexpr int BOX_BYTES = BQ * 128;         // one 128-row x 128-B box
  constexpr uint32_t S_COL0 = 0, S_COL1 = 128, O_COL0 = 256, O_COL1 = 384;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2];
  __shared__ uint64_t s_full[2], p_full[2], o_full[2];
  __shared__ uint64_t x_bar[2][4];          // max / sum exchange between the two threads of a row, per q tile and quadrant
  __shared__ float x_val[2][2][BQ];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem;                       // 2 tiles
  uint8_t* sK = sQ + 2 * TILE_BYTES;        // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;        // 2 stages

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_blk = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int q0 = q_blk * 2 * BQ;

  int kv_valid = p.Skv;
  if (p.kv_len != nullptr) kv_valid = min(kv_valid, p.kv_len[batch]);
  if (kv_valid < 1) kv_valid = 1;
  const int n_kv = (kv_valid + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 256);
      for (int qd = 0; qd < 4; ++qd) mbar_init(&x_bar[s][qd], 64);
      mbar_init(&o_full[s], 1);
    }
    abort_s = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp < 4) {
    setmaxnreg_dec<CTRL_REGS>();
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    if (warp == 0 && (MODE != 0 || lane == 0)) {
      // ----------------------------- TMA producer -----------------------------
      if (ctl_issuer<MODE>()) {
        mbar_expect_tx(&q_full, 2 * TILE_BYTES);
        for (int t = 0; t < 2; ++t)
          for (int d = 0; d < DBOX; ++d)
            tma_load_4d(sQ + t * TILE_BYTES + d * BOX_BYTES, &maps.q, &q_full, d * 64, q0 + t * BQ, head, batch);
      }
      ctl_rejoin<MODE>();
      bool ok = true;
      uint64_t* last_bar = &q_full;
      uint32_t last_par = 0;
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t par = (j >> 1) & 1;
        if (!ctl_wait<MODE>(&k_empty[st], par ^ 1u, &abort_s, lane)) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 11, j);
          ok = false;
          break;
        }
        if (ctl_issuer<MODE>()) {
          mbar_expect_tx(&k_full[st], TILE_BYTES);
          for (int d = 0; d < DBOX; ++d)
            tma_load_4d(sK + st * TILE_BYTES + d * BOX_BYTES, &maps.k, &k_full[st], d * 64, j * BKV, head, batch);
        }
        ctl_rejoin<MODE>();
        last_bar = &k_full[st];
        last_par = par;
        if (!ctl_wait<MODE>(&v_empty[st], par ^ 1u, &abort_s, lane)) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 12, j);
          ok = false;
          break;
        }
        if (ctl_issuer<MODE>()) {
          mbar_expect_tx(&v_full[st], TILE_BYTES);
          for (int d = 0; d < DBOX; ++d)
            tma_load_4d(sV + st * TILE_BYTES + d * BOX_BYTES, &maps.v, &v_full[st], d * 64, j * BKV, head, batch);
        }
        ctl_rejoin<MODE>();
        last_bar = &v_full[st];
        last_par = par;
      }
      if (!ok) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(last_bar, last_par) && globaltimer_ns() - t0 < 5000000ull) {
        }
      }
    } else if (warp == 1 && (MODE != 0 || lane == 0)) {
      // ----------------------------- UMMA issuer ------------------------------
      // (Two issuing warps, one per q tile, were measured slower: the issuers block on the tensor pipe's short queue, so
      // issue time is execution time, and two of them only contend.) Descriptors are built once; each MMA adds a constant
      // to the address field.
      constexpr uint32_t idesc_s = make_idesc(1, UMMA_BF16, UMMA_BF16, 0, 0, BQ, BKV);
      constexpr uint32_t idesc_pv = make_idesc(1, UMMA_BF16, UMMA_BF16, 0, 1, BQ, DH);
      const uint32_t s_tmem[2] = {tmem_base + S_COL0, tmem_base + S_COL1};
      const uint32_t o_tmem[2] = {tmem_base + O_COL0, tmem_base + O_COL1};
      const uint64_t q_desc[2] = {make_desc_kmajor_sw128(smem_u32(sQ)), make_desc_kmajor_sw128(smem_u32(sQ + TILE_BYTES))};
      const uint64_t k_desc[2] = {make_desc_kmajor_sw128(smem_u32(sK)), make_desc_kmajor_sw128(smem_u32(sK + TILE_BYTES))};
      const uint64_t v_desc[2] = {make_desc_mnmajor_sw128(smem_u32(sV), BOX_BYTES),
                                  make_desc_mnmajor_sw128(smem_u32(sV + TILE_BYTES), BOX_BYTES)};
      // both helpers run in the issuing lane only
      auto issue_s = [&](int t, int st) {
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = static_cast<uint32_t>((kk / 4) * BOX_BYTES + (kk % 4) * 32) >> 4;
          umma_f16_ss(s_tmem[t], q_desc[t] + off, k_desc[st] + off, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int st, bool first) {
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          umma_f16_ts(o_tmem[t], s_tmem[t] + kk * 8, v_desc[st] + static_cast<uint32_t>((kk * 2048) >> 4), idesc_pv,
                      (first && kk == 0) ? 0u : 1u);
        umma_commit(&o_full[t]);
      };
      bool ok = ctl_wait<MODE>(&q_full, 0, &abort_s, lane) && ctl_wait<MODE>(&k_full[0], 0, &abort_s, lane);
      if (!ok && lane == 0) report_status(p.status, STATUS_TIMEOUT, 21, 0);
      if (ok) {
        tc_fence_after();
        if (ctl_issuer<MODE>()) {
          issue_s(0, 0);
          issue_s(1, 0);
          umma_commit(&k_empty[0]);
        }
        ctl_rejoin<MODE>();
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t par = (j >> 1) & 1;
        const bool more = (j + 1 < n_kv);
        const int st_n = (j + 1) & 1;
        const uint32_t par_n = ((j + 1) >> 1) & 1;
        if (!ctl_wait<MODE>(&v_full[st], par, &abort_s, lane) || (more && !ctl_wait<MODE>(&k_full[st_n], par_n, &abort_s, lane))) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 22, j);
          ok = false;
          break;
        }
        for (int t = 0; t < 2; ++t) {
          if (!ctl_wait<MODE>(&p_full[t], j & 1, &abort_s, lane)) {
            if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 23 + t, j);
            ok = false;
            break;
          }
          if (tracing && lane == 0 && (j * 2 + t) < p.trace_len) p.trace[0 * p.trace_len + j * 2 + t] = clock64();
          tc_fence_after();
          if (ctl_issuer<MODE>()) {
            issue_pv(t, st, j == 0);
            if (more) issue_s(t, st_n);
            if (t == 1) {
              umma_commit(&v_empty[st]);
              if (more) umma_commit(&k_empty[st_n]);
            }
          }
          ctl_rejoin<MODE>();
          if (tracing && lane == 0 && (j * 2 + t) < p.trace_len) p.trace[1 * p.trace_len + j * 2 + t] = clock64();
        }
        if (!ok) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- softmax warps: two threads per query row ---------------
    // Warps 4-7 own key columns 0..63 of every S tile (and output columns 0..Dh/2-1), warps 8-11 the other half; the two
    // threads of a row sit in warps with the same TMEM lane quadrant. Both q tiles are processed by the same threads in
    // turn, so tile 0's P V and next Q K^T run on the tensor core while all eight warps do tile 1's softmax and vice
    // versa: the exponentials of one tile are spread over all four special-function units with two warps each. Per kv
    // tile the two halves exchange their row maxima through shared memory (an mbarrier of 64 arrivals per tile and
    // quadrant, bounded wait), so both use the same exponent reference and take the same rescale decisions; the row sums
    // stay partial and are added once at the end.
    setmaxnreg_inc<SOFTMAX_REGS>();
    const int half = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale_log2;
    constexpr int OH = DH / 2;                 // output columns per thread
    float m_used[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    bool ok = true;

    // max / sum exchange between the two threads of a row
    auto exchange = [&](int t, float mine, uint32_t parity, float& other) -> bool {
      x_val[t][half][row_in_tile] = mine;
      mbar_arrive(&x_bar[t][quad]);
      const bool got = mbar_wait(&x_bar[t][quad], parity, &abort_s);
      other = x_val[t][half ^ 1][row_in_tile];
      return got;
    };

    for (int j = 0; ok && j < n_kv; ++j) {
      const int kv0 = j * BKV + half * 64;
      const bool tail = j * BKV + BKV > kv_valid;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t s_tile = tmem_base + lane_addr + (t ? S_COL1 : S_COL0);
        const uint32_t o_addr = tmem_base + lane_addr + (t ? O_COL1 : O_COL0) + half * OH;
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, &abort_s));
        if (!ok) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 31 + t, j);
          break;
        }
        tc_fence_after();
        const bool tr = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 4 && lane == 0 &&
                        4 * j + 3 < p.trace_len;
        if (tr) p.trace[(2 + t) * p.trace_len + 4 * j] = clock64();
        uint32_t s0[32], s1[32];
        tmem_ld_32x32b_x32(s_tile + half * 64, s0);
        tmem_ld_32x32b_x32(s_tile + half * 64 + 32, s1);
        tmem_wait_ld();
        if (tr) p.trace[(2 + t) * p.trace_len + 4 * j + 1] = clock64();
        if (tail) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (kv0 + i >= kv_valid) s0[i] = 0xff800000u;        // -inf
            if (kv0 + 32 + i >= kv_valid) s1[i] = 0xff800000u;
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {                 // three-input maxima: 32 instructions for 64 values
          mx0 = fmax3(mx0, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(s0[i + 2]), __uint_as_float(s0[i + 3]));
          mx2 = fmax3(mx2, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
          mx3 = fmax3(mx3, __uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3]));
        }
        float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
        float other;
        ok = __all_sync(0xffffffffu, exchange(t, mx, j & 1, other));
        if (!ok) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 37 + t, j);
          break;
        }
        mx = fmaxf(mx, other);                     // the row's maximum over all 128 keys of the tile, same in both halves
        if (tr) p.trace[(2 + t) * p.trace_len + 4 * j + 2] = clock64();
        if (j == 0) {
          m_used[t] = mx;
        } else {
          // lazy rescale: raise the exponent reference only when a row outgrew it by more than 2^8
          const bool need = mx > m_used[t] + 8.0f;
          if (__any_sync(0xffffffffu, need)) {
            ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], (j - 1) & 1, &abort_s));
            if (!ok) {
              if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 33 + t, j);
              break;
            }
            tc_fence_after();
            const float alpha = need ? exp2f(m_used[t] - mx) : 1.0f;
            if (need) m_used[t] = mx;
            l_run[t] *= alpha;
#pragma unroll
            for (int c = 0; c < OH / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(o_addr + c * 32, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32b_x32(o_addr + c * 32, r);
            }
            tmem_wait_st();
          }
        }
        const float mref = m_used[t];
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
        const float2 sl2_2 = make_float2(sl2, sl2), nm2 = make_float2(-mref, -mref);
        auto emit = [&](const uint32_t (&sv)[32], int c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            // Four scores per step as two packed pairs (scale and reference in one packed fma each). The special-function
            // unit (16 results per clock per SM) bounds a loop of plain exponentials, so the odd elements of every
            // POLY_EVERY-th group go through the packed polynomial on the FMA pipe instead.
            const float2 x01 = ffma2(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sl2_2, nm2);
            const float2 x23 = ffma2(make_float2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])), sl2_2, nm2);
            const float2 a = make_float2(ex2_approx(x01.x), ex2_approx(x23.x));
            float2 b;
            if (POLY_EVERY > 0 && ((i >> 2) % POLY_EVERY) == POLY_EVERY - 1) b = ex2_poly2(make_float2(x01.y, x23.y));
            else b = make_float2(ex2_approx(x01.y), ex2_approx(x23.y));
            sum_a = fadd2(sum_a, a);
            sum_b = fadd2(sum_b, b);
            pk[i >> 1] = pack_bf16x2(a.x, b.x);
            pk[(i >> 1) + 1] = pack_bf16x2(a.y, b.y);
          }
          // P (bf16) of this half: 32 TMEM columns at half * 32 of the tile's S region; both halves have loaded their S
          // values before the exchange above, so nothing still needed is overwritten
          tmem_st_32x32b_x16(s_tile + half * 32 + c * 16, pk);
        };
        emit(s0, 0);
        emit(s1, 1);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[t]);
        if (tr) p.trace[(2 + t) * p.trace_len + 4 * j + 3] = clock64();
        l_run[t] += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
      }
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (!ok) break;
      const uint32_t o_addr = tmem_base + lane_addr + (t ? O_COL1 : O_COL0) + half * OH;
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], (n_kv - 1) & 1, &abort_s));
      if (!ok) {
        if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 35 + t, n_kv);
        break;
      }
      tc_fence_after();
      float l_other;
      ok = __all_sync(0xffffffffu, exchange(t, l_run[t], n_kv & 1, l_other));
      if (!ok) {
        if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 39 + t, n_kv);
        break;
      }
      const float l_tot = l_run[t] + l_other;
      const float inv_l = 1.f / l_tot;
      // The normalised rows go through shared memory (this tile's Q buffer: every S = Q K^T has completed by now, 32 rows
      // per quadrant) so that the global stores are whole rows: DH / 8 lanes x 16 bytes per row instead of one 16-byte
      // piece of 32 different rows per instruction. That matters most when the rows are routed into a peer's memory.
      constexpr int CH = DH / 8;                       // 16-byte chunks per output row
      uint8_t* stage = sQ + t * TILE_BYTES + quad * (32 * DH * 2);
      uint4* my_row = reinterpret_cast<uint4*>(stage + lane * (DH * 2));
#pragma unroll
      for (int c = 0; c < OH / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(o_addr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(r[i + 0]) * inv_l, __uint_as_float(r[i + 1]) * inv_l);
          w.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l);
          w.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l);
          w.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l);
          my_row[(half * (CH / 2) + c * 4 + (i >> 3)) ^ (lane & (CH - 1))] = w;
        }
      }
      // both halves of the quadrant's 32 rows are staged (a rendezvous only: the exchange slots are not written again, the
      // partner may still be reading the row sum left there)
      mbar_arrive(&x_bar[t][quad]);
      ok = __all_sync(0xffffffffu, mbar_wait(&x_bar[t][quad], (n_kv + 1) & 1, &abort_s));
      if (!ok) {
        if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 41 + t, n_kv);
        break;
      }
      const int chunk = lane % CH;
#pragma unroll 4
      for (int i = 0; i < CH / 2; ++i) {
        const int rl = half * 16 + i * (32 / CH) + lane / CH;          // this warp copies 16 of the quadrant's 32 rows
        const int tk = q0 + t * BQ + quad * 32 + rl;
        if (tk >= p.Sq) continue;
        __nv_bfloat16* obase = p.o;
        long long otok = tk;
        if (p.route_rows_a > 0) {
          if (tk < p.route_split) {
            const int owner = tk / p.route_rows_a;
            obase = reinterpret_cast<__nv_bfloat16*>(p.o_route_a[owner]);
            otok = tk - owner * p.route_rows_a;
          } else {
            const int u = tk - p.route_split;
            const int owner = u / p.route_rows_b;
            obase = reinterpret_cast<__nv_bfloat16*>(p.o_route_b[owner]);
            otok = u - owner * p.route_rows_b;
          }
        }
        __nv_bfloat16* orow = obase + batch * p.o_strides[0] + otok * p.o_strides[1] + head * p.o_strides[2];
        *reinterpret_cast<uint4*>(orow + chunk * 8) =
            reinterpret_cast<const uint4*>(stage + rl * (DH * 2))[chunk ^ (rl & (CH - 1))];
      }
      const int tok = q0 + t * BQ + row_in_tile;
      if (half == 0 && p.lse != nullptr && tok < p.Sq)
        p.lse[(static_cast<long long>(batch) * p.H + head) * p.Sq + tok] = (m_used[t] + log2f(l_tot)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DH, int MODE, int POLY_EVERY>
static int launch_attn(const AttnMaps& maps, const AttnParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * BQ * DH * 2 + 1024;
  auto kern = attention_fwd_kernel<DH, MODE, POLY_EVERY>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  dim3 grid((p.Sq + 2 * BQ - 1) / (2 * BQ), p.H, p.B);
  kern<<<grid, ATT_THREADS, SMEM, st>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

static int make_bshd_map(CUtensorMap* m, const void* ptr, int B, int S, int H, int Dh, const long long* strides) {
  // dims innermost first: (d, seq, head, batch)
  int64_t ext[4] = {Dh, S, H, B};
  int64_t str[4] = {2, strides[1] * 2, strides[2] * 2, strides[0] * 2};
  int box[4] = {64, 128, 1, 1};
  return mdb_make_tmap(m, ptr, 2, 4, ext, str, box, 1);
}

}  // namespace mdb

extern "C" int mdb_attention_fwd(const MdbAttnArgs* a, cudaStream_t st) {
  using namespace mdb;
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Skv <= 0) return -1;
  if (a->Dh != 128 && a->Dh != 64) return -2;
  for (int i = 0; i < 3; ++i) {
    if ((a->q_strides[i] % 8) || (a->k_strides[i] % 8) || (a->v_strides[i] % 8) || (a->o_strides[i] % 8)) return -3;
  }
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       (a->route_rows_a > 0 ? 0 : reinterpret_cast<uintptr_t>(a->o))) & 15)
    return -4;
  AttnMaps maps;
  int r = make_bshd_map(&maps.q, a->q, a->B, a->Sq, a->H, a->Dh, a->q_strides);
  if (r) return 1000 + r;
  r = make_bshd_map(&maps.k, a->k, a->B, a->Skv, a->H, a->Dh, a->k_strides);
  if (r) return 2000 + r;
  r = make_bshd_map(&maps.v, a->v, a->B, a->Skv, a->H, a->Dh, a->v_strides);
  if (r) return 3000 + r;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.o = reinterpret_cast<__nv_bfloat16*>(a->o);
  p.lse = a->lse;
  p.kv_len = a->kv_len;
  p.B = a->B; p.H = a->H; p.Sq = a->Sq; p.Skv = a->Skv;
  for (int i = 0; i < 3; ++i) p.o_strides[i] = a->o_strides[i];
  p.scale_log2 = a->scale * 1.4426950408889634f;
  {
    static int mode = -1;
    if (mode < 0) {
      const char* e = getenv("MDB200_ATTN_EXP_POLY");
      mode = (e != nullptr && e[0] >= '0' && e[0] <= '4') ? e[0] - '0' : MDB_ATTN_POLY_DEFAULT;
    }
    p.exp_poly = mode;
  }
  p.status = a->status;
  for (int i = 0; i < 8; ++i) {
    p.o_route_a[i] = a->o_route_a[i];
    p.o_route_b[i] = a->o_route_b[i];
  }
  p.route_rows_a = a->route_rows_a;
  p.route_split = a->route_rows_a > 0 ? (a->o_route_b[0] ? a->route_split : a->Sq) : 0;
  p.route_rows_b = a->route_rows_b > 0 ? a->route_rows_b : 1;
  p.trace = g_attn_trace;
  p.trace_len = g_attn_trace_len;
  static int issue_mode = -1;
  if (issue_mode < 0) {
    const char* e = getenv("MDB200_ATTN_ISSUE");     // 0 / 1 / 2: see ctl_wait; measurement switch
    issue_mode = (e != nullptr && e[0] >= '0' && e[0] <= '1') ? e[0] - '0' : MDB_ATTN_ISSUE_DEFAULT;
  }
  // p.exp_poly: 0 = every exponential on the special-function unit; N = one exponential in 2N as a polynomial on the FMA pipe
  // (MDB200_ATTN_EXP_POLY, default MDB_ATTN_POLY_DEFAULT)
#define MDB_ATTN_GO(DH_, MODE_)                                                     \
  do {                                                                              \
    if (p.exp_poly == 1) return launch_attn<DH_, MODE_, 1>(maps, p, st);            \
    if (p.exp_poly == 2) return launch_attn<DH_, MODE_, 2>(maps, p, st);            \
    if (p.exp_poly == 4) return launch_attn<DH_, MODE_, 4>(maps, p, st);            \
    return launch_attn<DH_, MODE_, 0>(maps, p, st);                                 \
  } while (0)
  if (a->Dh == 128) {
    if (issue_mode == 0) MDB_ATTN_GO(128, 0);
    MDB_ATTN_GO(128, 1);
  }
  if (issue_mode == 0) MDB_ATTN_GO(64, 0);
  MDB_ATTN_GO(64, 1);
#undef MDB_ATTN_GO
}

// Debugging aid: the next forward launches write a clock64 time line of CTA (0, 0, 0) into `trace` (device memory,
// [4][len] int64: 0 = MMA issuer saw P ready per (kv tile, q tile); 1 = MMA issuer done issuing; 2 / 3 = softmax warpgroup
// 0 / 1: S seen, S loaded, maximum done, P published per kv tile). NULL switches it off.
extern "C" void mdb_attention_set_trace(long long* trace, int len) {
  mdb::g_attn_trace = trace;
  mdb::g_attn_trace_len = len;
}

MDB_DEFINE_WAIT_LIMIT_SETTER(mdb_set_wait_limit_attn_fwd)
