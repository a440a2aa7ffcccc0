// Persistent warp-specialised GEMM for sm_100a: TMA (128-byte swizzle) -> shared memory ring ->
// tcgen05.mma with the accumulator in TMEM (double buffered, so the epilogue of tile i overlaps the
// main loop of tile i+1) -> tcgen05.ld epilogue with fused bias / activation / gated residual /
// paired (SwiGLU, GEGLU) / dequant-scale math and direct vector stores.
//
//   out[M,N] = epi( sum_seg  A_seg[M,K_seg] * B_seg[N,K_seg]^T )
//
// Up to three K segments share one accumulator. That is how a LoRA up-projection (A2 = x*down^T,
// B2 = up), a split input (FLUX single-block linear2 over [attn | gelu(mlp)]) or a beta=1
// accumulate are folded into one launch without a concat.
//
// Operand majors: K-major (row-major [rows,K], the forward layout of x and of nn.Linear weights) and
// MN-major (the same buffers read transposed: dx = dY*W uses W MN-major, dW = dY^T*x uses both).
// Element kinds: bf16 (kind::f16) and fp8 e4m3 (kind::f8f6f4, scales applied in the epilogue).
//
// Covers the role of the reference's cuBLAS call + bias/cast kernels (serenitymojo/ops/linear.mojo:40-180,182,404),
// its GEMM backward calls (serenitymojo/ops/linalg_backward.mojo:99-124) and its weight-only fp8 kernel
// (serenitymojo/ops/fp8_gemm.mojo:28-73).
#include "common.cuh"
#include "gemm_api.h"

#include <cudaTypedefs.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace mdb {

constexpr int BM = 128;
constexpr int BK_BYTES = 128;  // one swizzle atom row: 64 bf16 or 128 fp8
constexpr int GATHER_STAGES = 2;          // shared-memory stages of the fused all-gather (bulk copies)
constexpr int GATHER_PIECE = 16384;       // bytes per stage
constexpr int NUM_THREADS = 224;  // warps: 0 TMA, 1 UMMA issue, 2-5 epilogue, 6 peer gather (all-gather fused GEMM)
constexpr int CONV_TW = 16, CONV_TH = 8;  // conv mode: one M tile = 8 rows x 16 columns of output pixels

struct alignas(64) GemmMaps {
  CUtensorMap a[MDB_GEMM_MAX_SEG];
  CUtensorMap b[MDB_GEMM_MAX_SEG];
};

struct GemmParams {
  int M, N;
  int num_seg;
  int kblocks[MDB_GEMM_MAX_SEG];
  int pair_offset;  // paired mode (>0): second half of the B tile comes from rows n0 + pair_offset
  int act;          // MDB_ACT_*
  int act_on_second;  // paired mode: 0 -> act(first)*second (SwiGLU), 1 -> first*act(second) (GEGLU)
  float alpha;
  const float* row_scale;          // [M] or null
  const float* col_scale;          // [N(+pair)] or null
  const __nv_bfloat16* bias;       // [N(+pair)] or null
  const __nv_bfloat16* residual;   // [M, ld_res] or null
  const __nv_bfloat16* gate;       // [groups, gate_stride] or null; group = row / rows_per_group
  int ld_res, gate_stride, rows_per_group;
  void* out;
  int ld_out;
  int out_fp32;
  int accumulate_out;  // out += result (fp32 out only)
  int* status;
  long long* prof;  // optional [grid, 8] cycle counters (profiling builds of the caller)
  long long* trace;  // optional per-K-block time line of CTAs 0 and 1: [2 CTAs][3 roles][trace_len] clock64 values
  int trace_len;
  // peer-routed output (sequence-parallel all-to-all in the epilogue): see MdbGemmArgs
  void* route_out[MDB_GEMM_MAX_PEERS];
  int route_owner_cols, route_part_cols, route_row_offset, route_rows_per_batch, route_batch_rows;
  int route_split, route_row_offset_b;
  // all-gather fused into the GEMM (gather_world > 1): operand A (gather_operand 0) or B (1) lives in a local
  // buffer of `gather_world` equal row chunks; chunk r is rank r's shard. Warp 6 of every CTA copies its slice of
  // each remote chunk from the owner's memory (peer loads) and bumps ready[chunk]; the TMA producer waits for
  // ready[chunk] == gridDim.x before it loads a tile of that chunk. Tiles are visited local chunk first.
  const void* gather_src[MDB_GEMM_MAX_PEERS];
  void* gather_dst;
  int* gather_ready;
  long long gather_chunk_bytes;
  int gather_world, gather_rank, gather_operand, gather_chunk_rows;
  // reduce-scatter fused into the epilogue (route_owner_cols == 0 && reduce_rows_per_owner > 0): fp32 partial
  // results are added (red.global.add) into the row owner's fp32 buffer route_out[row / reduce_rows_per_owner]
  int reduce_rows_per_owner;
  int split_k;           // > 1: the K range of the single segment is cut into split_k parts, one work item each;
                         // parts are added into a zero-initialised fp32 output with red.global.add (skinny GEMMs)
  int reduce_src_rank;   // staged bf16 variant: slot of the owner's staging buffer this rank writes
  // implicit-GEMM convolution (conv_taps > 0): A is an NHWC image read through a 4-D tensor map, one 16x8 pixel
  // patch per M tile, one shifted box per filter tap; rows outside the image are skipped by the epilogue
  int conv_taps, conv_kw, conv_pad_h, conv_pad_w, conv_h, conv_w, conv_tiles_h, conv_tiles_w, conv_cblocks, conv_tiles_m;
};

__device__ __forceinline__ float apply_act_rt(int act, float x) {
  switch (act) {
    case MDB_ACT_GELU_TANH: return gelu_tanh_f(x);
    case MDB_ACT_SILU: return silu_f(x);
    case MDB_ACT_GELU_ERF: return gelu_erf_f(x);
    default: return x;
  }
}

// 32 consecutive bf16 -> fp32 (64 bytes, 16-byte aligned)
__device__ __forceinline__ void load32_bf16(const __nv_bfloat16* p, float (&f)[32]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 u = q[i];
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[i * 8 + 0] = a.x; f[i * 8 + 1] = a.y; f[i * 8 + 2] = b.x; f[i * 8 + 3] = b.y;
    f[i * 8 + 4] = c.x; f[i * 8 + 5] = c.y; f[i * 8 + 6] = d.x; f[i * 8 + 7] = d.y;
  }
}
__device__ __forceinline__ void load32_f32(const float* p, float (&f)[32]) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 u = q[i];
    f[i * 4 + 0] = u.x; f[i * 4 + 1] = u.y; f[i * 4 + 2] = u.z; f[i * 4 + 3] = u.w;
  }
}

template <int ACT>
__device__ __forceinline__ void act32(float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (ACT == MDB_ACT_GELU_TANH) v[j] = gelu_tanh_f(v[j]);
    if (ACT == MDB_ACT_SILU) v[j] = silu_f(v[j]);
    if (ACT == MDB_ACT_GELU_ERF) v[j] = gelu_erf_f(v[j]);
  }
}
__device__ __forceinline__ void act32_rt(int act, float (&v)[32]) {
  // the flag is tested once per 32 values; each case is a tight unrolled loop
  if (act == MDB_ACT_GELU_TANH) act32<MDB_ACT_GELU_TANH>(v);
  else if (act == MDB_ACT_SILU) act32<MDB_ACT_SILU>(v);
  else if (act == MDB_ACT_GELU_ERF) act32<MDB_ACT_GELU_ERF>(v);
}

// Where a 32-column slab of output row `row` starting at column `col0` goes. Plain GEMM: the local output.
// Routed mode: columns are (part, owner, local) blocks; the slab is stored into the owner rank's buffer at
// row  batch * route_batch_rows + route_row_offset + row_in_batch  and column  part * owner_cols + local.
__device__ __forceinline__ void* out_slab_ptr(const GemmParams& p, int row, int col0, int esz) {
  if (p.reduce_rows_per_owner > 0) {
    const int owner = row / p.reduce_rows_per_owner;
    size_t orow = static_cast<size_t>(row - owner * p.reduce_rows_per_owner);
    if (!p.out_fp32) orow += static_cast<size_t>(p.reduce_src_rank) * p.reduce_rows_per_owner;
    return reinterpret_cast<char*>(p.route_out[owner]) + (orow * p.ld_out + col0) * esz;
  }
  if (p.route_owner_cols <= 0)
    return reinterpret_cast<char*>(p.out) + (static_cast<size_t>(row) * p.ld_out + col0) * esz;
  const int part = col0 / p.route_part_cols;
  const int within = col0 - part * p.route_part_cols;
  const int owner = within / p.route_owner_cols;
  const int lcol = part * p.route_owner_cols + (within - owner * p.route_owner_cols);
  const int b = row / p.route_rows_per_batch;
  const int rin = row - b * p.route_rows_per_batch;
  const int off = (p.route_split > 0 && rin >= p.route_split) ? p.route_row_offset_b + (rin - p.route_split) : p.route_row_offset + rin;
  const size_t orow = static_cast<size_t>(b) * p.route_batch_rows + off;
  return reinterpret_cast<char*>(p.route_out[owner]) + (orow * p.ld_out + lcol) * esz;
}

// Ragged edge (fewer than 32 columns left, or an unaligned pointer): scalar, rarely taken.
__device__ __noinline__ void epilogue_row32_slow(const GemmParams& p, int row, int col0, int ncols, const uint32_t* r,
                                                 const uint32_t* r2, bool paired) {
  const float rs = (p.row_scale ? p.row_scale[row] : 1.f) * p.alpha;
  for (int j = 0; j < ncols; ++j) {
    const int col = col0 + j;
    float x = __uint_as_float(r[j]) * rs;
    if (p.col_scale) x *= p.col_scale[col];
    if (p.bias) x += __bfloat162float(p.bias[col]);
    if (paired) {
      float y = __uint_as_float(r2[j]) * rs;
      if (p.col_scale) y *= p.col_scale[col + p.pair_offset];
      if (p.bias) y += __bfloat162float(p.bias[col + p.pair_offset]);
      x = p.act_on_second ? x * apply_act_rt(p.act, y) : apply_act_rt(p.act, x) * y;
    } else {
      x = apply_act_rt(p.act, x);
    }
    if (p.gate) x *= __bfloat162float(p.gate[static_cast<size_t>(row / p.rows_per_group) * p.gate_stride + col]);
    if (p.residual) x += __bfloat162float(p.residual[static_cast<size_t>(row) * p.ld_res + col]);
    if (p.out_fp32) {
      float* o = reinterpret_cast<float*>(out_slab_ptr(p, row, col0, 4)) + j;
      if (p.reduce_rows_per_owner > 0 || p.split_k > 1) atomicAdd(o, x);   // fp32 reduce mode / split-K parts
      else *o = p.accumulate_out ? *o + x : x;
    } else {
      reinterpret_cast<__nv_bfloat16*>(out_slab_ptr(p, row, col0, 2))[j] = __float2bfloat16_rn(x);
    }
  }
}

// One 32-column slab of one output row. r[] holds the raw accumulators (r2[] the paired half).
// stage_row (optional): this lane's 256-byte row of the warp's shared-memory staging buffer; the packed bf16 slab then
// goes there (16-byte chunks stage_chunk0 .. +3, XOR-swizzled by the lane so that neither the row-wise writes nor the
// later chunk-wise reads conflict) instead of to global memory.
__device__ __forceinline__ void epilogue_row32(const GemmParams& p, int row, int col0, const uint32_t (&r)[32],
                                               const uint32_t (&r2)[32], bool paired, bool aligned,
                                               uint4* stage_row = nullptr, int stage_chunk0 = 0, int swz = 0) {
  if (row >= p.M || col0 >= p.N) return;
  const int ncols = min(32, p.N - col0);
  if (ncols < 32 || !aligned) {
    // copies live in local memory only on this branch, so the fast path keeps its accumulators in registers
    uint32_t t0[32], t1[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      t0[j] = r[j];
      t1[j] = paired ? r2[j] : 0u;
    }
    epilogue_row32_slow(p, row, col0, ncols, t0, t1, paired);
    return;
  }
  float v[32];
  const float rs = (p.row_scale ? p.row_scale[row] : 1.f) * p.alpha;
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * rs;
  if (p.col_scale) {
    float t[32];
    load32_f32(p.col_scale + col0, t);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= t[j];
  }
  if (p.bias) {
    float t[32];
    load32_bf16(p.bias + col0, t);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += t[j];
  }
  if (paired) {
    float w[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = __uint_as_float(r2[j]) * rs;
    if (p.col_scale) {
      float t[32];
      load32_f32(p.col_scale + col0 + p.pair_offset, t);
#pragma unroll
      for (int j = 0; j < 32; ++j) w[j] *= t[j];
    }
    if (p.bias) {
      float t[32];
      load32_bf16(p.bias + col0 + p.pair_offset, t);
#pragma unroll
      for (int j = 0; j < 32; ++j) w[j] += t[j];
    }
    if (p.act_on_second) act32_rt(p.act, w); else act32_rt(p.act, v);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= w[j];
  } else if (p.act != MDB_ACT_NONE) {
    act32_rt(p.act, v);
  }
  if (p.gate) {
    float t[32];
    load32_bf16(p.gate + static_cast<size_t>(row / p.rows_per_group) * p.gate_stride + col0, t);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= t[j];
  }
  if (p.residual) {
    float t[32];
    load32_bf16(p.residual + static_cast<size_t>(row) * p.ld_res + col0, t);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += t[j];
  }
  if (p.out_fp32) {
    float4* o = reinterpret_cast<float4*>(out_slab_ptr(p, row, col0, 4));
    if (p.reduce_rows_per_owner > 0 || p.split_k > 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                     "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                     : "memory");
    } else if (p.accumulate_out) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 old = o[j];
        o[j] = make_float4(old.x + v[4 * j], old.y + v[4 * j + 1], old.z + v[4 * j + 2], old.w + v[4 * j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  } else {
    uint4* o = stage_row ? stage_row : reinterpret_cast<uint4*>(out_slab_ptr(p, row, col0, 2));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 t;
      t.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
      t.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
      t.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
      t.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
      o[stage_row ? ((stage_chunk0 + j) ^ swz) : j] = t;
    }
  }
}

// Epilogue of one accumulator tile for one warp (its 32 TMEM lanes = 32 output rows). bf16 outputs whose tile lies fully
// inside the matrix go through an 8 KB per-warp staging buffer in shared memory, 128 columns at a time: every lane packs
// its row's slabs into the buffer, then the warp stores whole 256-byte row segments (16 lanes x 16 bytes per row, two
// rows per instruction). Local stores become full cache lines and peer-routed stores (sequence-parallel scatter, staged
// reduce-scatter) cross NVLink as 256-byte writes instead of 64-byte fragments of 32 different rows. Everything else
// (fp32 outputs, ragged edges, unaligned pointers) keeps the direct per-lane stores.
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t taddr, int pair_col_off, int row, int n0,
                                              int out_cols, bool paired, bool aligned, uint8_t* stage_warp, int lane) {
  const bool staged = stage_warp != nullptr && aligned && !p.out_fp32 && (out_cols & 127) == 0 && n0 + out_cols <= p.N;
  if (!staged) {
#pragma unroll 1
    for (int c = 0; c < out_cols / 32; ++c) {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(taddr + c * 32, r0);
      if (paired) tmem_ld_32x32b_x32(taddr + pair_col_off + c * 32, r1);
      tmem_wait_ld();
      epilogue_row32(p, row, n0 + c * 32, r0, r1, paired, aligned);
    }
    return;
  }
  uint4* my_row = reinterpret_cast<uint4*>(stage_warp + lane * 256);
  const int swz = lane & 15;
#pragma unroll 1
  for (int g = 0; g < out_cols / 128; ++g) {
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(taddr + g * 128 + c * 32, r0);
      if (paired) tmem_ld_32x32b_x32(taddr + pair_col_off + g * 128 + c * 32, r1);
      tmem_wait_ld();
      epilogue_row32(p, row, n0 + g * 128 + c * 32, r0, r1, paired, true, my_row, c * 4, swz);
    }
    __syncwarp();
    const int chunk = lane & 15;
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const int rl = 2 * i + (lane >> 4);                       // row of the warp this lane copies in this pass
      const int rr = __shfl_sync(0xffffffffu, row, rl);         // its global output row (p.M or more: not stored)
      const uint4 v = reinterpret_cast<const uint4*>(stage_warp + rl * 256)[chunk ^ (rl & 15)];
      if (rr < p.M) *reinterpret_cast<uint4*>(out_slab_ptr(p, rr, n0 + g * 128 + chunk * 8, 2)) = v;
    }
    __syncwarp();
  }
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Tile -> (m block, n block). Plain GEMM: m fastest. With a fused all-gather the gathered operand's blocks are
// visited starting at the local chunk (already present), then in the order the gather warps fetch the peers.
__device__ __forceinline__ int tile_m_index(const GemmParams& p, int tile, int tiles_m, int tiles_n) {
  if (p.gather_world > 1 && p.gather_operand == 1) return tile % tiles_m;
  int m = tile % tiles_m;
  if (p.gather_world > 1) {
    const int shift = (p.gather_rank * p.gather_chunk_rows) / BM;
    m = (m + shift) % tiles_m;
  }
  return m;
}
__device__ __forceinline__ int tile_n_index(const GemmParams& p, int tile, int tiles_m, int tiles_n) {
  int n = tile / tiles_m;
  if (p.gather_world > 1 && p.gather_operand == 1) {
    const int bn_rows = (p.N + tiles_n - 1) / tiles_n;
    const int shift = (p.gather_rank * p.gather_chunk_rows) / max(bn_rows, 1);
    n = (n + shift) % tiles_n;
  }
  return n;
}

// KIND: 0 = bf16 operands (kind::f16), 1 = fp8 e4m3 operands (kind::f8f6f4)
template <int BN, int STAGES, bool A_MN, bool B_MN, int KIND>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
  constexpr int A_BYTES = BM * BK_BYTES;
  constexpr int B_BYTES = BN * BK_BYTES;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  constexpr int KSTEPS = 4;  // 128-byte rows / 32 bytes per UMMA K step
  static_assert(!(KIND == 1 && (A_MN || B_MN)), "fp8 operands are K-major only");

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ uint64_t gather_bar[GATHER_STAGES];

  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);
    }
    for (int s = 0; s < GATHER_STAGES; ++s) mbar_init(&gather_bar[s], 1);
    abort_s = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < p.num_seg; ++s) {
      tma_prefetch_desc(&maps.a[s]);
      tma_prefetch_desc(&maps.b[s]);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  const int tiles_m = p.conv_taps > 0 ? p.conv_tiles_m : (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + (p.pair_offset > 0 ? BN / 2 : BN) - 1) / (p.pair_offset > 0 ? BN / 2 : BN);
  const int num_tiles = tiles_m * tiles_n;
  const int splits = p.split_k > 1 ? p.split_k : 1;
  const int num_items = num_tiles * splits;          // work item = (tile, K part); part = item / num_tiles
  int total_kb = 0;
  for (int s = 0; s < p.num_seg; ++s) total_kb += p.kblocks[s];
  // K blocks [kb_lo, kb_hi) of segment 0 that work item `item` covers (the whole segment without split-K)
  auto kb_lo_of = [&](int item) { return splits > 1 ? static_cast<int>(static_cast<long long>(item / num_tiles) * p.kblocks[0] / splits) : 0; };
  auto kb_hi_of = [&](int item) { return splits > 1 ? static_cast<int>(static_cast<long long>(item / num_tiles + 1) * p.kblocks[0] / splits) : p.kblocks[0]; };
  constexpr int K_ELEMS = (KIND == 0) ? 64 : 128;  // elements per 128-byte row

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    // The whole warp runs the loop (waits included) and elect.sync picks the lane that issues: tcgen05 / TMA instructions
    // issued from a convergent warp cost about 120 cycles each, from inside a one-lane branch about 190 (measured), which
    // is more than the 128 cycles a 128 x 256 x 16 MMA takes.
    {
      int stage = 0;
      uint32_t phase = 0;
      int last_stage = -1;
      uint32_t last_phase = 0;
      bool ok = true;
      long long t_wait = 0;
      unsigned chunk_seen = 1u << p.gather_rank;   // chunks whose arrival this CTA has already observed
      int n_trace = 0;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int tile = item % num_tiles;
        const int m0 = tile_m_index(p, tile, tiles_m, tiles_n) * BM;
        const int nblk = tile_n_index(p, tile, tiles_m, tiles_n);
        const int n0 = p.pair_offset > 0 ? nblk * (BN / 2) : nblk * BN;
        if (p.gather_world > 1) {
          // every chunk this tile touches must have landed (a tile may straddle two chunks)
          const int r0 = p.gather_operand == 0 ? m0 : n0;
          const int r1 = r0 + (p.gather_operand == 0 ? BM : BN) - 1;
          const int c_lo = min(r0 / p.gather_chunk_rows, p.gather_world - 1);
          const int c_hi = min(r1 / p.gather_chunk_rows, p.gather_world - 1);
          for (int c = c_lo; ok && c <= c_hi; ++c) {
            if (chunk_seen & (1u << c)) continue;
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            bool mine = true;
            while (ld_acquire_gpu(p.gather_ready + c) < static_cast<int>(gridDim.x)) {
              if ((++spins & 0xffu) == 0 && (abort_s || globaltimer_ns() - t0 > MDB_WAIT_LIMIT_NS)) {
                abort_s = 1;
                mine = false;
                break;
              }
            }
            if (!__all_sync(0xffffffffu, mine)) {
              if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 5, c);
              ok = false;
              break;
            }
            chunk_seen |= 1u << c;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");   // peer-copied bytes -> visible to the TMA reads
        }
        for (int s = 0; ok && s < p.num_seg; ++s) {
          const int kb_begin = s == 0 ? kb_lo_of(item) : 0, kb_end = s == 0 ? kb_hi_of(item) : p.kblocks[s];
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            const long long tw0 = p.prof ? clock64() : 0;
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_s))) {
              if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 1, stage);
              ok = false;
              break;
            }
            if (p.prof) t_wait += clock64() - tw0;
            if (p.trace && lane == 0 && blockIdx.x < 2 && n_trace < p.trace_len) p.trace[(blockIdx.x * 3 + 0) * p.trace_len + n_trace++] = clock64();
            uint8_t* sa = smem + stage * STAGE_BYTES;
            uint8_t* sb = sa + A_BYTES;
            int k0 = kb * K_ELEMS;
            if (elect_one()) {
              mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
              if (p.conv_taps > 0) {
                // tile -> (image, patch row, patch col); k block -> (filter tap, channel block)
                const int mt = tile % tiles_m;
                const int tw = mt % p.conv_tiles_w, th = (mt / p.conv_tiles_w) % p.conv_tiles_h;
                const int img = mt / (p.conv_tiles_w * p.conv_tiles_h);
                const int tap = kb / p.conv_cblocks, cb = kb - tap * p.conv_cblocks;
                const int kh = tap / p.conv_kw, kw = tap - kh * p.conv_kw;
                tma_load_4d(sa, &maps.a[s], &full_bar[stage], cb * K_ELEMS, tw * CONV_TW + kw - p.conv_pad_w,
                            th * CONV_TH + kh - p.conv_pad_h, img);
                k0 = (tap * p.conv_cblocks + cb) * K_ELEMS;
              } else if (!A_MN) {
                tma_load_2d(sa, &maps.a[s], &full_bar[stage], k0, m0);
              } else {
                // boxes [64 m-elements][64 k-rows], 8 KB each
                tma_load_2d(sa, &maps.a[s], &full_bar[stage], m0, k0);
                tma_load_2d(sa + 8192, &maps.a[s], &full_bar[stage], m0 + 64, k0);
              }
              if (!B_MN) {
                constexpr int HALF_ROWS = BN / 2;
                const int n1 = p.pair_offset > 0 ? n0 + p.pair_offset : n0 + HALF_ROWS;
                tma_load_2d(sb, &maps.b[s], &full_bar[stage], k0, n0);
                tma_load_2d(sb + HALF_ROWS * BK_BYTES, &maps.b[s], &full_bar[stage], k0, n1);
              } else {
#pragma unroll
                for (int j = 0; j < BN / 64; ++j)
                  tma_load_2d(sb + j * 8192, &maps.b[s], &full_bar[stage], n0 + j * 64, k0);
              }
            }
            __syncwarp();
            last_stage = stage;
            last_phase = phase;
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (p.prof && lane == 0) p.prof[blockIdx.x * 8 + 1] = t_wait;
      if (!ok && last_stage >= 0) {
        // abandoned: let the copies already in flight land before the CTA goes away (bounded)
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&full_bar[last_stage], last_phase) && globaltimer_ns() - t0 < 5000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer --------------------------------
    // whole warp in the loop, elect.sync for the issuing lane (see the producer)
    {
      constexpr uint32_t idesc =
          (KIND == 0) ? make_idesc(1, UMMA_BF16, UMMA_BF16, A_MN ? 1u : 0u, B_MN ? 1u : 0u, BM, BN)
                      : make_idesc(1, UMMA_E4M3, UMMA_E4M3, 0u, 0u, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long t_full = 0, t_tempty = 0;
      int n_trace = 0;
      const long long t_begin = p.prof ? clock64() : 0;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x, ++it) {
        const int item_kb = splits > 1 ? kb_hi_of(item) - kb_lo_of(item) : total_kb;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        const long long te0 = p.prof ? clock64() : 0;
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, &abort_s))) {
          if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 2, acc);
          break;
        }
        if (p.prof) t_tempty += clock64() - te0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < item_kb; ++kb) {
          const long long tf0 = p.prof ? clock64() : 0;
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, &abort_s))) {
            if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 3, stage);
            ok = false;
            break;
          }
          if (p.prof) t_full += clock64() - tf0;
          if (p.trace && lane == 0 && blockIdx.x < 2 && n_trace < p.trace_len) p.trace[(blockIdx.x * 3 + 1) * p.trace_len + n_trace++] = clock64();
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint64_t da = A_MN ? make_desc_mnmajor_sw128(sa, 8192) : make_desc_kmajor_sw128(sa);
          const uint64_t db = B_MN ? make_desc_mnmajor_sw128(sb, 8192) : make_desc_kmajor_sw128(sb);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
              // K-major: 32 bytes along the row per step; MN-major: 16 K-rows of 128 B per step
              const uint64_t a_k = da + static_cast<uint64_t>(A_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              const uint64_t b_k = db + static_cast<uint64_t>(B_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              if (KIND == 0)
                umma_f16_ss(d_tmem, a_k, b_k, idesc, (kb | k) != 0 ? 1u : 0u);
              else
                umma_f8_ss(d_tmem, a_k, b_k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);  // smem slot free once these UMMAs have read it
            if (kb == item_kb - 1) umma_commit(&tfull_bar[acc]);
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (p.prof && lane == 0) {
        p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
        p.prof[blockIdx.x * 8 + 2] = t_full;
        p.prof[blockIdx.x * 8 + 3] = t_tempty;
        p.prof[blockIdx.x * 8 + 6] = it;
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------- peer gather (all-gather fused GEMM) --------
    if (p.gather_world > 1 && lane == 0) {
      // One thread streams this CTA's share of every peer chunk through two 16 KB shared-memory stages with bulk copies:
      // peer memory -> shared (completion on an mbarrier), shared -> the local gathered buffer (bulk group). 32 KB are in
      // flight per CTA, which keeps NVLink busy from all SMs together; nothing passes through registers.
      uint8_t* gs = smem + STAGES * STAGE_BYTES;
      const long long pieces = (p.gather_chunk_bytes + GATHER_PIECE - 1) / GATHER_PIECE;
      uint32_t ph[GATHER_STAGES] = {0, 0};
      bool ok = true;
      for (int i = 1; i < p.gather_world && ok; ++i) {
        const int c = (p.gather_rank + i) % p.gather_world;
        const char* src = reinterpret_cast<const char*>(p.gather_src[c]);
        char* dst = reinterpret_cast<char*>(p.gather_dst) + c * p.gather_chunk_bytes;
        const long long mine = blockIdx.x < pieces ? (pieces - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        auto piece_off = [&](long long k) { return (static_cast<long long>(blockIdx.x) + k * gridDim.x) * GATHER_PIECE; };
        auto piece_len = [&](long long k) {
          const long long rem = p.gather_chunk_bytes - piece_off(k);
          return static_cast<uint32_t>(rem < GATHER_PIECE ? rem : GATHER_PIECE);
        };
        auto issue = [&](long long k) {
          const int sgi = static_cast<int>(k % GATHER_STAGES);
          mbar_expect_tx(&gather_bar[sgi], piece_len(k));
          bulk_load_g2s(gs + sgi * GATHER_PIECE, src + piece_off(k), piece_len(k), &gather_bar[sgi]);
        };
        long long issued = 0;
        for (; issued < mine && issued < GATHER_STAGES; ++issued) issue(issued);
        for (long long k = 0; k < mine; ++k) {
          const int sgi = static_cast<int>(k % GATHER_STAGES);
          if (!mbar_wait(&gather_bar[sgi], ph[sgi], &abort_s)) {
            report_status(p.status, STATUS_TIMEOUT, 70, c);
            ok = false;
            // bounded drain of the loads still in flight (jobs k .. issued-1), so that nothing lands in shared memory
            // after this CTA has left
            for (long long j = k; j < issued; ++j) {
              const int sj = static_cast<int>(j % GATHER_STAGES);
              const uint64_t t0 = globaltimer_ns();
              while (!mbar_try_wait(&gather_bar[sj], ph[sj]) && globaltimer_ns() - t0 < MDB_WAIT_LIMIT_NS) {}
            }
            break;
          }
          ph[sgi] ^= 1;
          bulk_store_s2g(dst + piece_off(k), gs + sgi * GATHER_PIECE, piece_len(k));
          tma_store_commit();
          if (issued < mine) {
            tma_store_wait_read<0>();                      // the stage has been read out: it may be refilled
            issue(issued++);
          }
        }
        tma_store_wait<0>();                               // this CTA's share of chunk c is in the gathered buffer
        if (!ok) break;
        __threadfence();
        atomicAdd(p.gather_ready + c, 1);
      }
    }
  } else {
    // ------------------------------- epilogue (4 warps) -------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const bool paired = p.pair_offset > 0;
    // the vector epilogue needs 16-byte aligned rows in every tensor it touches (columns advance in 64-byte steps)
    const int esz = p.out_fp32 ? 4 : 2;
    bool aligned = ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(static_cast<size_t>(p.ld_out) * esz)) & 15) == 0;
    if (p.bias) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.bias) | static_cast<uintptr_t>(p.pair_offset * 2)) & 15) == 0;
    if (p.col_scale) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.col_scale) | static_cast<uintptr_t>(p.pair_offset * 4)) & 15) == 0;
    if (p.gate) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.gate) | static_cast<uintptr_t>(p.gate_stride * 2)) & 15) == 0;
    if (p.residual) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.residual) | static_cast<uintptr_t>(static_cast<size_t>(p.ld_res) * 2)) & 15) == 0;
    int it = 0;
    long long t_twait = 0, t_work = 0;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x, ++it) {
      const int tile = item % num_tiles;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = tile_m_index(p, tile, tiles_m, tiles_n) * BM;
      const int nblk = tile_n_index(p, tile, tiles_m, tiles_n);
      const int n0 = paired ? nblk * (BN / 2) : nblk * BN;
      const long long tq0 = p.prof ? clock64() : 0;
      // warp-uniform decision: the TMEM loads below are warp-collective
      const bool got = __all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, &abort_s));
      if (!got) {
        if (lane == 0) report_status(p.status, STATUS_TIMEOUT, 4, acc);
        break;
      }
      tc_fence_after();
      const long long tq1 = p.prof ? clock64() : 0;
      t_twait += tq1 - tq0;
      if (p.trace && blockIdx.x < 2 && warp == 2 && lane == 0 && 2 * it + 1 < p.trace_len) p.trace[(blockIdx.x * 3 + 2) * p.trace_len + 2 * it] = clock64();
      int row = m0 + quad * 32 + lane;
      if (p.conv_taps > 0) {
        const int mt = tile % tiles_m;
        const int tw = mt % p.conv_tiles_w, th = (mt / p.conv_tiles_w) % p.conv_tiles_h;
        const int img = mt / (p.conv_tiles_w * p.conv_tiles_h);
        const int r = quad * 32 + lane;
        const int oh = th * CONV_TH + r / CONV_TW, ow = tw * CONV_TW + r % CONV_TW;
        row = (oh < p.conv_h && ow < p.conv_w) ? (img * p.conv_h + oh) * p.conv_w + ow : p.M;  // p.M = skipped
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const int out_cols = paired ? BN / 2 : BN;
      // the staging buffers share their 32 KB with the stages of the fused all-gather, which therefore stores directly
      uint8_t* stage_warp = p.gather_world > 1 ? nullptr : smem + STAGES * STAGE_BYTES + quad * 8192;
      epilogue_tile(p, taddr, BN / 2, row, n0, out_cols, paired, aligned, stage_warp, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (p.prof) t_work += clock64() - tq1;
      if (p.trace && blockIdx.x < 2 && warp == 2 && lane == 0 && 2 * it + 1 < p.trace_len) p.trace[(blockIdx.x * 3 + 2) * p.trace_len + 2 * it + 1] = clock64();
    }
    if (p.prof && warp == 2 && lane == 0) {
      p.prof[blockIdx.x * 8 + 4] = t_twait;
      p.prof[blockIdx.x * 8 + 5] = t_work;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------
// CTA-pair variant: one 256 x 256 output tile per cluster of two CTAs (tcgen05 cta_group::2). Each CTA stages its
// own 128 rows of A and its own 128 rows of B per K block (32 KB instead of the 48 KB a lone 128 x 256 CTA needs for
// the same MMA time), so the shared-memory fill rate, which bounds the one-CTA kernel on DiT shapes, drops by a third
// and the ring is 6 stages deep. The even CTA issues the MMAs for both; each CTA reads its own 128 x 256 fp32
// accumulator from its own TMEM and runs the same fused epilogue. bf16 operands, any operand majors, paired (GLU)
// mode, routed / staged-reduce epilogues; no fused gather, convolution or split-K (those stay on the one-CTA kernel).
// ---------------------------------------------------------------------------------
constexpr int PAIR_THREADS = 192;  // warps: 0 TMA, 1 UMMA issue (leader only), 2-5 epilogue

template <int STAGES, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
  constexpr int BN = 256;               // accumulator columns per CTA (the whole tile width)
  constexpr int BNH = 128;              // B rows staged by one CTA
  constexpr int A_BYTES = BM * BK_BYTES;
  constexpr int B_BYTES = BNH * BK_BYTES;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;
  constexpr int KSTEPS = 4;
  constexpr int K_ELEMS = 64;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES];    // used in the leader: both CTAs' loads of a stage have landed
  __shared__ uint64_t empty_bar[STAGES];   // in each CTA: the MMAs that read this stage are done
  __shared__ uint64_t tfull_bar[2];        // in each CTA: accumulator complete
  __shared__ uint64_t tempty_bar[2];       // used in the leader: 8 epilogue warps (4 per CTA) have drained the accumulator
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 8);
    }
    abort_s = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_s, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < p.num_seg; ++s) {
      tma_prefetch_desc(&maps.a[s]);
      tma_prefetch_desc(&maps.b[s]);
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // the peer's barriers exist before anything is sent to them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t peer_abort = mapa_shared(smem_u32(&abort_s), rank ^ 1u);

  const bool paired = p.pair_offset > 0;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + (paired ? BNH : BN) - 1) / (paired ? BNH : BN);
  const int num_tiles = tiles_m * tiles_n;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  int total_kb = 0;
  for (int s = 0; s < p.num_seg; ++s) total_kb += p.kblocks[s];

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------
    // whole warp in the loop, elect.sync for the issuing lane (see the one-CTA kernel)
    {
      int stage = 0;
      uint32_t phase = 0;
      int last_stage = -1;
      bool ok = true;
      long long t_wait = 0;
      int n_trace = 0;
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
        const int m0 = (tile % tiles_m) * (2 * BM) + static_cast<int>(rank) * BM;
        const int nblk = tile / tiles_m;
        // this CTA's 128 rows of B: the lower / upper half of the tile, or in paired mode the first / second operand
        const int n0 = paired ? nblk * BNH + (leader ? 0 : p.pair_offset) : nblk * BN + static_cast<int>(rank) * BNH;
        for (int s = 0; ok && s < p.num_seg; ++s) {
          for (int kb = 0; kb < p.kblocks[s]; ++kb) {
            const long long tw0 = p.prof ? clock64() : 0;
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_s))) {
              if (lane == 0) {
                report_status(p.status, STATUS_TIMEOUT, 21, stage);
                st_shared_cluster_u32(peer_abort, 1u);
              }
              ok = false;
              break;
            }
            if (p.prof) t_wait += clock64() - tw0;
            if (p.trace && lane == 0 && blockIdx.x < 2 && n_trace < p.trace_len) p.trace[(blockIdx.x * 3 + 0) * p.trace_len + n_trace++] = clock64();
            uint8_t* sa = smem + stage * STAGE_BYTES;
            uint8_t* sb = sa + A_BYTES;
            const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0u);
            const int k0 = kb * K_ELEMS;
            if (elect_one()) {
              if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
              if (!A_MN) {
                tma_load_2d_pair(sa, &maps.a[s], bar, k0, m0);
              } else {
                tma_load_2d_pair(sa, &maps.a[s], bar, m0, k0);
                tma_load_2d_pair(sa + 8192, &maps.a[s], bar, m0 + 64, k0);
              }
              if (!B_MN) {
                tma_load_2d_pair(sb, &maps.b[s], bar, k0, n0);
              } else {
                tma_load_2d_pair(sb, &maps.b[s], bar, n0, k0);
                tma_load_2d_pair(sb + 8192, &maps.b[s], bar, n0 + 64, k0);
              }
            }
            __syncwarp();
            last_stage = stage;
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (p.prof && lane == 0) p.prof[blockIdx.x * 8 + 1] = t_wait;
      if (!ok && last_stage >= 0) {
        // abandoned: give the copies already in flight time to land before the CTA goes away (bounded)
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer (leader CTA only) --------------
    if (leader) {
      constexpr uint32_t idesc = make_idesc(1, UMMA_BF16, UMMA_BF16, A_MN ? 1u : 0u, B_MN ? 1u : 0u, 2 * BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long t_full = 0, t_tempty = 0;
      int n_trace = 0;
      const long long t_begin = p.prof ? clock64() : 0;
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        const long long te0 = p.prof ? clock64() : 0;
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, &abort_s))) {
          if (lane == 0) {
            report_status(p.status, STATUS_TIMEOUT, 22, acc);
            st_shared_cluster_u32(peer_abort, 1u);
          }
          break;
        }
        if (p.prof) t_tempty += clock64() - te0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < total_kb; ++kb) {
          const long long tf0 = p.prof ? clock64() : 0;
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, &abort_s))) {
            if (lane == 0) {
              report_status(p.status, STATUS_TIMEOUT, 23, stage);
              st_shared_cluster_u32(peer_abort, 1u);
            }
            ok = false;
            break;
          }
          if (p.prof) t_full += clock64() - tf0;
          if (p.trace && lane == 0 && blockIdx.x < 2 && n_trace < p.trace_len) p.trace[(blockIdx.x * 3 + 1) * p.trace_len + n_trace++] = clock64();
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint64_t da = A_MN ? make_desc_mnmajor_sw128(sa, 8192) : make_desc_kmajor_sw128(sa);
          const uint64_t db = B_MN ? make_desc_mnmajor_sw128(sb, 8192) : make_desc_kmajor_sw128(sb);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
              const uint64_t a_k = da + static_cast<uint64_t>(A_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              const uint64_t b_k = db + static_cast<uint64_t>(B_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              umma_f16_ss_pair(d_tmem, a_k, b_k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit_pair(&empty_bar[stage], 3);   // the stage is free in both CTAs once these MMAs have read it
            if (kb == total_kb - 1) umma_commit_pair(&tfull_bar[acc], 3);
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (p.prof && lane == 0) {
        p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
        p.prof[blockIdx.x * 8 + 2] = t_full;
        p.prof[blockIdx.x * 8 + 3] = t_tempty;
        p.prof[blockIdx.x * 8 + 6] = it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (4 warps per CTA) -----------------
    const int quad = warp & 3;
    const int esz = p.out_fp32 ? 4 : 2;
    bool aligned = ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(static_cast<size_t>(p.ld_out) * esz)) & 15) == 0;
    if (p.bias) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.bias) | static_cast<uintptr_t>(p.pair_offset * 2)) & 15) == 0;
    if (p.col_scale) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.col_scale) | static_cast<uintptr_t>(p.pair_offset * 4)) & 15) == 0;
    if (p.gate) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.gate) | static_cast<uintptr_t>(p.gate_stride * 2)) & 15) == 0;
    if (p.residual) aligned = aligned && ((reinterpret_cast<uintptr_t>(p.residual) | static_cast<uintptr_t>(static_cast<size_t>(p.ld_res) * 2)) & 15) == 0;
    int it = 0;
    long long t_twait = 0, t_work = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = (tile % tiles_m) * (2 * BM) + static_cast<int>(rank) * BM;
      const int nblk = tile / tiles_m;
      const int n0 = paired ? nblk * BNH : nblk * BN;
      const long long tq0 = p.prof ? clock64() : 0;
      const bool got = __all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, &abort_s));
      if (!got) {
        if (lane == 0) {
          report_status(p.status, STATUS_TIMEOUT, 24, acc);
          st_shared_cluster_u32(peer_abort, 1u);
        }
        break;
      }
      tc_fence_after();
      const long long tq1 = p.prof ? clock64() : 0;
      t_twait += tq1 - tq0;
      if (p.trace && blockIdx.x < 2 && warp == 2 && lane == 0 && 2 * it + 1 < p.trace_len) p.trace[(blockIdx.x * 3 + 2) * p.trace_len + 2 * it] = clock64();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const int out_cols = paired ? BNH : BN;
      epilogue_tile(p, taddr, BNH, row, n0, out_cols, paired, aligned, smem + STAGES * STAGE_BYTES + quad * 8192, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0u));
      if (p.prof) t_work += clock64() - tq1;
      if (p.trace && blockIdx.x < 2 && warp == 2 && lane == 0 && 2 * it + 1 < p.trace_len) p.trace[(blockIdx.x * 3 + 2) * p.trace_len + 2 * it + 1] = clock64();
    }
    if (p.prof && warp == 2 && lane == 0) {
      p.prof[blockIdx.x * 8 + 4] = t_twait;
      p.prof[blockIdx.x * 8 + 5] = t_work;
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // neither CTA frees TMEM or leaves while its partner may still signal or read
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(f);
  }
  return fn;
}

}  // namespace mdb

extern "C" int mdb_make_tmap(void* out_map, const void* ptr, int elem_bytes, int rank, const int64_t* extents,
                             const int64_t* strides_bytes, const int* box, int swizzle128) {
  auto fn = mdb::get_encode_fn();
  if (!fn) return -1;
  // The encode call is a driver-API entry and needs a current context. A thread that has not made a runtime call yet
  // (an autograd worker whose first node is one of our backward kernels) has none: bind the primary context once.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = static_cast<cuuint64_t>(extents[i]);
    bdim[i] = static_cast<cuuint32_t>(box[i]);
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = static_cast<cuuint64_t>(strides_bytes[i]);
  }
  CUtensorMapDataType dt = elem_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), dt, rank, const_cast<void*>(ptr), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

namespace mdb {

template <int BN, int STAGES, bool A_MN, bool B_MN, int KIND>
static int launch_variant(const GemmMaps& maps, const GemmParams& p, int num_sms, cudaStream_t stream) {
  constexpr int STAGE_BYTES = BM * BK_BYTES + BN * BK_BYTES;
  // operand ring + 32 KB that serve as the epilogue's staging buffers (4 warps x 8 KB) or, with a fused all-gather, as its
  // two bulk-copy stages
  constexpr int SMEM_GATHER = STAGES * STAGE_BYTES + 1024 + GATHER_STAGES * GATHER_PIECE;
  static_assert(GATHER_STAGES * GATHER_PIECE == 4 * 8192, "staging buffers and gather stages share one region");
  static_assert(SMEM_GATHER <= 227 * 1024, "pipeline + staging exceed the shared memory of an SM");
  const int SMEM = SMEM_GATHER;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, A_MN, B_MN, KIND>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_GATHER);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  const int tiles_m = p.conv_taps > 0 ? p.conv_tiles_m : (p.M + BM - 1) / BM;
  const int bn_eff = p.pair_offset > 0 ? BN / 2 : BN;
  const int tiles_n = (p.N + bn_eff - 1) / bn_eff;
  if (p.split_k > 1 && p.kblocks[0] < p.split_k) return -10;
  int grid = tiles_m * tiles_n * (p.split_k > 1 ? p.split_k : 1);
  if (grid > num_sms) grid = num_sms;
  if (grid < 1) return 0;
  kern<<<grid, NUM_THREADS, SMEM, stream>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

// How many CTA pairs the device can hold at once: an SM whose partner in the same TPC is not available cannot host half
// a pair, so the number differs from chip to chip. A persistent grid must not exceed it (surplus pairs would run their
// whole tile list after the others finish) and the tile-shape choice uses it as the pair kernel's width.
template <int STAGES, bool A_MN, bool B_MN>
__global__ void gemm_tcgen05_pair_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p);

static int pair_capacity(int num_sms) {
  static int cached = 0;
  if (cached > 0) return cached;
  constexpr int SMEM = 6 * (BM * BK_BYTES + 128 * BK_BYTES) + 4 * 8192 + 1024;
  auto kern = gemm_tcgen05_pair_kernel<6, false, false>;
  int n = 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) == cudaSuccess) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(num_sms & ~1), 1, 1);
    cfg.blockDim = dim3(PAIR_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
  }
  cudaGetLastError();
  if (n < 1 || n > num_sms / 2) n = num_sms / 2;
  cached = n;
  return cached;
}

template <int STAGES, bool A_MN, bool B_MN>
static int launch_pair_variant(const GemmMaps& maps, const GemmParams& p, int num_sms, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (BM * BK_BYTES + 128 * BK_BYTES) + 4 * 8192 + 1024;   // ring + epilogue staging (4 warps x 8 KB)
  static_assert(SMEM <= 227 * 1024, "pipeline exceeds the shared memory of an SM");
  auto kern = gemm_tcgen05_pair_kernel<STAGES, A_MN, B_MN>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + (p.pair_offset > 0 ? 128 : 256) - 1) / (p.pair_offset > 0 ? 128 : 256);
  const int max_pairs = pair_capacity(num_sms);
  int clusters = tiles_m * tiles_n;
  if (clusters > max_pairs) clusters = max_pairs;
  if (clusters < 1) return 0;
  kern<<<2 * clusters, PAIR_THREADS, SMEM, stream>>>(maps, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mdb

extern "C" int mdb_gemm_pair_capacity(int num_sms) { return mdb::pair_capacity(num_sms > 0 ? num_sms : mdb::device_sm_count()); }

// MDB200_GEMM_PAIR=0 keeps every automatically tiled GEMM on the one-CTA kernel (A/B measurements); default: choose.
static int pair_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("MDB200_GEMM_PAIR");
    mode = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return mode;
}

extern "C" int mdb_gemm_launch(const MdbGemmArgs* a, cudaStream_t stream) {
  using namespace mdb;
  if (a->M <= 0 || a->N <= 0 || a->num_seg < 1 || a->num_seg > MDB_GEMM_MAX_SEG) return -2;
  const int eb = a->kind == 1 ? 1 : 2;
  const int k_elems = BK_BYTES / eb;
  const bool paired = a->pair_offset > 0;
  const int sms = a->num_sms > 0 ? a->num_sms : device_sm_count();
  int bn = a->bn;
  // bn == 512 asks for the CTA-pair kernel (256 x 256 tile over two SMs); it shares the tensor maps of the 128 x 256 tile
  const bool pair_ok = a->kind == 0 && a->conv_taps <= 0 && a->gather_world <= 1 && a->split_k <= 1;
  bool use_pair = bn == 512 && pair_ok;
  if (bn == 512) bn = 256;
  const bool auto_tile = bn != 64 && bn != 128 && bn != 256;
  if (bn != 64 && bn != 128 && bn != 256) {
    // default tile choice: 128x256 unless the narrower 128x128 tile fills the machine noticeably better
    // (fewer idle SMs in the last wave); 128x64 only for very skinny outputs
    const int tm = (a->M + BM - 1) / BM;
    auto wave_eff = [&](int w) {
      const long long tiles = static_cast<long long>(tm) * ((a->N + w - 1) / w);
      const long long waves = (tiles + sms - 1) / sms;
      return static_cast<double>(tiles) / static_cast<double>(waves * sms);
    };
    bn = 256;
    if (!paired && wave_eff(128) > 1.12 * wave_eff(256)) bn = 128;
    if (!paired && a->N <= 64) bn = 64;
  }
  if (paired && bn != 256) bn = 256;
  if (auto_tile && pair_ok && a->M > BM && pair_mode() != 0) {
    // CTA pair (256 x 256 tile on two SMs) or lone CTAs? Compare waves x time per tile. A lone CTA's 128 x 256 tile moves
    // 96 KB through shared memory per K block (48 KB written by TMA, 48 KB read by the tensor core): 726 cycles measured,
    // bound by the 128 B/clk of shared memory. A pair tile moves 64 KB per SM and runs at the tensor rate: 523 cycles.
    const int n_tile = paired ? 128 : 256;
    const long long t2 = static_cast<long long>((a->M + 2 * BM - 1) / (2 * BM)) * ((a->N + n_tile - 1) / n_tile);
    const int pairs = pair_capacity(sms);
    const long long w2 = (t2 + pairs - 1) / pairs;
    const long long t1 = static_cast<long long>((a->M + BM - 1) / BM) * ((a->N + (paired ? 128 : bn) - 1) / (paired ? 128 : bn));
    const long long w1 = (t1 + sms - 1) / sms;
    const double cost1 = static_cast<double>(w1) * (bn == 256 ? 1.0 : bn == 128 ? 0.55 : 0.32);
    const double cost2 = static_cast<double>(w2) * 0.72;
    if (cost2 <= cost1) {
      use_pair = true;
      bn = 256;
    }
  }
  GemmMaps maps;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M;
  p.N = a->N;
  p.num_seg = a->num_seg;
  const int n_rows_total = paired ? a->N + a->pair_offset : a->N;  // rows of B that exist
  for (int s = 0; s < a->num_seg; ++s) {
    const int64_t K = a->K[s];
    if (K <= 0) return -3;
    p.kblocks[s] = static_cast<int>((K + k_elems - 1) / k_elems);
    // A
    {
      int64_t ext[2], str[2];
      int box[2];
      if (a->conv_taps > 0) {
        if (s != 0 || a->a_mn || a->kind != 0) return -6;
        const int64_t cin = a->conv_cin;
        int64_t e4[4] = {cin, a->conv_w, a->conv_h, a->conv_n};
        int64_t s4[4] = {eb, cin * eb, a->conv_w * cin * eb, static_cast<int64_t>(a->conv_h) * a->conv_w * cin * eb};
        int b4[4] = {k_elems, CONV_TW, CONV_TH, 1};
        int r = mdb_make_tmap(&maps.a[s], a->A[s], eb, 4, e4, s4, b4, 1);
        if (r) return 1000 + r;
        p.kblocks[s] = a->conv_taps * static_cast<int>((cin + k_elems - 1) / k_elems);
      } else
      if (!a->a_mn) {  // [M rows][K] row-major
        ext[0] = K; ext[1] = a->M; str[0] = eb; str[1] = a->lda[s] * eb; box[0] = k_elems; box[1] = BM;
      } else {  // stored [K rows][M]
        ext[0] = a->M; ext[1] = K; str[0] = eb; str[1] = a->lda[s] * eb; box[0] = 64; box[1] = 64;
      }
      if (a->conv_taps <= 0) {
        int r = mdb_make_tmap(&maps.a[s], a->A[s], eb, 2, ext, str, box, 1);
        if (r) return 1000 + r;
      }
    }
    {
      int64_t ext[2], str[2];
      int box[2];
      if (!a->b_mn) {  // [N rows][K]
        ext[0] = K; ext[1] = n_rows_total; str[0] = eb; str[1] = a->ldb[s] * eb; box[0] = k_elems; box[1] = bn / 2;
      } else {  // stored [K rows][N]
        ext[0] = a->N; ext[1] = K; str[0] = eb; str[1] = a->ldb[s] * eb; box[0] = 64; box[1] = 64;
      }
      int r = mdb_make_tmap(&maps.b[s], a->B[s], eb, 2, ext, str, box, 1);
      if (r) return 2000 + r;
    }
  }
  p.pair_offset = a->pair_offset;
  p.act = a->act;
  p.act_on_second = a->act_on_second;
  p.alpha = a->alpha;
  p.row_scale = a->row_scale;
  p.col_scale = a->col_scale;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.gate = reinterpret_cast<const __nv_bfloat16*>(a->gate);
  p.ld_res = a->ld_res;
  p.gate_stride = a->gate_stride;
  p.rows_per_group = a->rows_per_group > 0 ? a->rows_per_group : 1;
  p.out = a->out;
  p.ld_out = a->ld_out;
  p.out_fp32 = a->out_fp32;
  p.accumulate_out = a->accumulate_out;
  p.status = a->status;
  p.prof = a->prof;
  p.trace = a->trace;
  p.trace_len = a->trace_len;
  for (int i = 0; i < MDB_GEMM_MAX_PEERS; ++i) p.route_out[i] = a->route_out[i];
  for (int i = 0; i < MDB_GEMM_MAX_PEERS; ++i) p.gather_src[i] = a->gather_src[i];
  p.gather_dst = a->gather_dst;
  p.gather_ready = a->gather_ready;
  p.gather_chunk_bytes = a->gather_chunk_bytes;
  p.gather_world = a->gather_world;
  p.gather_rank = a->gather_rank;
  p.gather_operand = a->gather_operand;
  p.gather_chunk_rows = a->gather_chunk_rows > 0 ? a->gather_chunk_rows : 1;
  p.reduce_rows_per_owner = a->reduce_rows_per_owner;
  if (a->gather_world > 1) {
    if (a->gather_ready == nullptr || a->gather_dst == nullptr || (a->gather_chunk_bytes & 15) || a->conv_taps > 0) return -8;
    cudaError_t e = cudaMemsetAsync(a->gather_ready, 0, sizeof(int) * MDB_GEMM_MAX_PEERS, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  p.reduce_src_rank = a->reduce_src_rank;
  p.split_k = a->split_k > 1 ? a->split_k : 1;
  if (p.split_k > 1) {
    // parts are summed with red.add into a zeroed fp32 output: no epilogue math, one K segment, plain output
    if (!a->out_fp32 || a->num_seg != 1 || a->bias || a->residual || a->gate || a->act || a->row_scale || a->col_scale ||
        a->pair_offset > 0 || a->conv_taps > 0 || a->gather_world > 1 || a->reduce_rows_per_owner > 0 ||
        a->route_owner_cols > 0 || a->accumulate_out)
      return -10;
  }
  if (a->reduce_rows_per_owner > 0 && !a->out_fp32 && (a->reduce_src_rank < 0 || a->reduce_src_rank >= MDB_GEMM_MAX_PEERS)) return -9;
  p.conv_taps = a->conv_taps;
  if (a->conv_taps > 0) {
    if (a->conv_cin % k_elems) return -7;
    p.conv_kw = a->conv_kw; p.conv_pad_h = a->conv_pad_h; p.conv_pad_w = a->conv_pad_w;
    p.conv_h = a->conv_h; p.conv_w = a->conv_w;
    p.conv_tiles_h = (a->conv_h + CONV_TH - 1) / CONV_TH;
    p.conv_tiles_w = (a->conv_w + CONV_TW - 1) / CONV_TW;
    p.conv_cblocks = a->conv_cin / k_elems;
    p.conv_tiles_m = a->conv_n * p.conv_tiles_h * p.conv_tiles_w;
  }
  p.route_owner_cols = a->route_owner_cols;
  p.route_part_cols = a->route_part_cols > 0 ? a->route_part_cols : a->N;
  p.route_row_offset = a->route_row_offset;
  p.route_rows_per_batch = a->route_rows_per_batch > 0 ? a->route_rows_per_batch : a->M;
  p.route_batch_rows = a->route_batch_rows;
  p.route_split = a->route_split;
  p.route_row_offset_b = a->route_row_offset_b;
  if (a->route_owner_cols > 0 && ((a->route_owner_cols % 32) || (p.route_part_cols % a->route_owner_cols))) return -5;

#define MDB_LAUNCH(BN_, ST_, AMN_, BMN_, KIND_) return launch_variant<BN_, ST_, AMN_, BMN_, KIND_>(maps, p, sms, stream)
  if (use_pair) {
    if (!a->a_mn && !a->b_mn) return launch_pair_variant<6, false, false>(maps, p, sms, stream);
    if (!a->a_mn && a->b_mn) return launch_pair_variant<6, false, true>(maps, p, sms, stream);
    if (a->a_mn && a->b_mn) return launch_pair_variant<6, true, true>(maps, p, sms, stream);
    return launch_pair_variant<6, true, false>(maps, p, sms, stream);
  }
  if (a->kind == 1) {
    if (a->a_mn || a->b_mn) return -4;
    if (bn == 256) MDB_LAUNCH(256, 4, false, false, 1);
    if (bn == 128) MDB_LAUNCH(128, 6, false, false, 1);
    MDB_LAUNCH(64, 8, false, false, 1);
  }
  if (!a->a_mn && !a->b_mn) {
    if (bn == 256) MDB_LAUNCH(256, 4, false, false, 0);
    if (bn == 128) MDB_LAUNCH(128, 6, false, false, 0);
    MDB_LAUNCH(64, 8, false, false, 0);
  }
  if (!a->a_mn && a->b_mn) {
    if (bn == 256) MDB_LAUNCH(256, 4, false, true, 0);
    if (bn == 128) MDB_LAUNCH(128, 6, false, true, 0);
    MDB_LAUNCH(64, 8, false, true, 0);
  }
  if (a->a_mn && a->b_mn) {
    if (bn == 256) MDB_LAUNCH(256, 4, true, true, 0);
    if (bn == 128) MDB_LAUNCH(128, 6, true, true, 0);
    MDB_LAUNCH(64, 8, true, true, 0);
  }
  if (bn == 256) MDB_LAUNCH(256, 4, true, false, 0);
  if (bn == 128) MDB_LAUNCH(128, 6, true, false, 0);
  MDB_LAUNCH(64, 8, true, false, 0);
#undef MDB_LAUNCH
}

MDB_DEFINE_WAIT_LIMIT_SETTER(mdb_set_wait_limit_gemm)
