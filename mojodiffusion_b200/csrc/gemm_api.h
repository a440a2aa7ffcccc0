// C interface of the tcgen05 GEMM (gemm_tcgen05.cu). Plain pointers and a stream: no framework types,
// so the kernels build in seconds and can be driven from C, ctypes or the torch binding alike.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MDB_GEMM_MAX_SEG 3
#define MDB_GEMM_MAX_PEERS 8

enum {
  MDB_ACT_NONE = 0,
  MDB_ACT_GELU_TANH = 1,
  MDB_ACT_SILU = 2,
  MDB_ACT_GELU_ERF = 3,
};

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MdbGemmArgs {
  int M, N;                        // output rows / cols (paired mode: N = cols of the combined output)
  int num_seg;                     // number of K segments accumulated into one output
  int64_t K[MDB_GEMM_MAX_SEG];     // contraction length per segment
  const void* A[MDB_GEMM_MAX_SEG]; // K-major: [M, lda]; MN-major (a_mn): [K, lda] read transposed
  const void* B[MDB_GEMM_MAX_SEG]; // K-major: [N, ldb]; MN-major (b_mn): [K, ldb] read transposed
  int64_t lda[MDB_GEMM_MAX_SEG];   // leading dimensions in elements (multiples of 8 for bf16, 16 for fp8)
  int64_t ldb[MDB_GEMM_MAX_SEG];
  int a_mn, b_mn;                  // operand majors
  int kind;                        // 0 bf16, 1 fp8 e4m3
  int bn;                          // 0 = choose, else 64 / 128 / 256
  int pair_offset;                 // >0: output col c combines B rows c and c + pair_offset (SwiGLU / GEGLU)
  int act, act_on_second;
  float alpha;
  const float* row_scale;          // [M] fp32 or null
  const float* col_scale;          // [N (+pair_offset)] fp32 or null
  const void* bias;                // bf16 [N (+pair_offset)] or null
  const void* residual;            // bf16 [M, ld_res] or null: out = residual + gate * value
  const void* gate;                // bf16 [groups, gate_stride] or null
  int ld_res, gate_stride, rows_per_group;
  void* out;                       // bf16 or fp32 [M, ld_out]
  int ld_out, out_fp32, accumulate_out;
  int num_sms;
  int* status;                     // device int[4], zero on entry; see common.cuh
  long long* prof;                 // optional device [grid, 8] cycle counters: total, producer wait, mma wait-full,
                                   // mma wait-accumulator, epilogue wait, epilogue work, tiles
  long long* trace;                // optional device [2 CTAs][3 roles][trace_len] clock64 time line (producer: stage free seen;
  int trace_len;                   // MMA issuer: operands seen; epilogue: accumulator seen / drained, alternating)
  // Peer-routed output (route_owner_cols > 0). The N output columns are `parts` of route_part_cols columns; inside
  // a part, consecutive blocks of route_owner_cols columns belong to ranks 0, 1, ... Block (part, owner) of output
  // row r is stored into route_out[owner] (that rank's buffer, leading dimension ld_out) at row
  // (r / route_rows_per_batch) * route_batch_rows + route_row_offset + r % route_rows_per_batch and column
  // part * route_owner_cols. This is the Ulysses head-scatter done by the projection's own epilogue.
  // Two row ranges per batch entry (route_split > 0): rows with r % route_rows_per_batch >= route_split go to
  // route_row_offset_b + (r % route_rows_per_batch - route_split) instead, so one GEMM over [text rows | image rows] of
  // every sample scatters both streams without slicing its input.
  void* route_out[MDB_GEMM_MAX_PEERS];
  int route_owner_cols, route_part_cols, route_row_offset, route_rows_per_batch, route_batch_rows;
  int route_split, route_row_offset_b;
  // All-gather fused GEMM (gather_world > 1): the operand selected by gather_operand (0 = A, 1 = B) is read from
  // the local buffer gather_dst = [gather_world chunks of gather_chunk_rows rows]; chunk r is fetched inside the
  // kernel from gather_src[r] (rank r's shard in peer memory, gather_chunk_bytes bytes); chunk gather_rank must
  // already be in place. gather_ready: local int[8] scratch (zeroed by the launcher).
  const void* gather_src[MDB_GEMM_MAX_PEERS];
  void* gather_dst;
  int* gather_ready;
  long long gather_chunk_bytes;
  int gather_world, gather_rank, gather_operand, gather_chunk_rows;
  // Reduce-scatter fused GEMM (reduce_rows_per_owner > 0, fp32 output): output row r is ADDED into
  // route_out[r / reduce_rows_per_owner] (that rank's fp32 [rows_per_owner, ld_out] buffer) with red.global.add.
  int reduce_rows_per_owner;
  // With a bf16 output (out_fp32 == 0) the reduce-scatter is STAGED instead: the row is stored (plain vector stores) into
  // slot reduce_src_rank of the owner's bf16 [world, rows_per_owner, ld_out] staging buffer; the owner sums the slots.
  int reduce_src_rank;
  // Split-K (split_k > 1): the K range is cut into split_k parts, each a separate work item of the persistent grid; the
  // parts are added (red.global.add) into the fp32 output, which the caller has zeroed. One K segment, no epilogue math.
  int split_k;
  // Implicit-GEMM convolution, stride 1 (conv_taps = KH*KW > 0): A[0] is an NHWC bf16 image [conv_n, conv_h, conv_w,
  // conv_cin] (conv_cin a multiple of 64), B[0] the filter [N, KH, KW, conv_cin] as a [N, KH*KW*conv_cin] matrix,
  // M = conv_n*conv_h*conv_w output pixels (output NHWC [.., N] with ld_out). Padding pad_h / pad_w is implicit:
  // taps that fall outside the image read zeros through the tensor map's out-of-range fill.
  int conv_taps, conv_kw, conv_pad_h, conv_pad_w, conv_n, conv_h, conv_w, conv_cin;
} MdbGemmArgs;

int mdb_gemm_launch(const MdbGemmArgs* args, cudaStream_t stream);

// number of two-CTA clusters of the 256 x 256 GEMM kernel the current device can hold at once (74 on a B200 whose 148 SMs
// all have their TPC partner, fewer otherwise)
int mdb_gemm_pair_capacity(int num_sms);

// rank-N tiled tensor map (extents/strides innermost first; strides_bytes[0] ignored)
int mdb_make_tmap(void* out_map, const void* ptr, int elem_bytes, int rank, const int64_t* extents,
                  const int64_t* strides_bytes, const int* box, int swizzle128);

#ifdef __cplusplus
}
#endif
