// C interface of the non-GEMM kernels of this package. Every function enqueues work on `st` and
// returns 0 on success, a negative number for a rejected argument, or a positive cudaError_t.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum {
  MDB_PW_IDENTITY = 0,
  MDB_PW_GELU_TANH = 1,
  MDB_PW_SILU = 2,
  MDB_PW_GELU_ERF = 3,
  MDB_PW_SIGMOID = 4,
  MDB_PW_RELU = 5,
  MDB_PW_TANH = 6,
};

#ifdef __cplusplus
extern "C" {
#endif

// one entry per tensor for the multi-tensor kernels (device array)
typedef struct MdbTensorEntry {
  void* param;
  void* grad;
  void* exp_avg;
  void* exp_avg_sq;
  void* shadow;      // optional bf16 copy of an fp32 master
  long long numel;
} MdbTensorEntry;

// ---- norm_rope.cu
int mdb_norm_modulate_fwd(const void* x, void* out, const void* weight, const void* bias, const void* scale,
                          const void* shift, float* stats, int rows, int D, int ldx, int ldo, int mod_stride,
                          int rows_per_group, float eps, int rms, cudaStream_t st);
int mdb_norm_modulate_bwd(const void* x, const void* dy, void* dx, const void* weight, const void* scale, int rows,
                          int D, int ldx, int lddy, int lddx, int mod_stride, int rows_per_group, float eps, int rms,
                          cudaStream_t st);
int mdb_qk_norm_rope(void* buf, const void* wq, const void* wk, const float* cosv, const float* sinv, long long tokens,
                     int tokens_per_batch, int H, int Dh, int row_stride, int q_off, int k_off, float eps,
                     int interleaved, int inverse, int do_norm, int rope_start, long long batch_stride, int pos_offset,
                     cudaStream_t st);
int mdb_qk_norm_rope_bwd(void* dbuf, const void* xbuf, const void* wq, const void* wk, const float* cosv,
                         const float* sinv, long long tokens, int tokens_per_batch, int H, int Dh, int row_stride,
                         int q_off, int k_off, float eps, int interleaved, int do_norm, int rope_start,
                         long long batch_stride, int pos_offset, cudaStream_t st);
int mdb_rope_table(const float* pos, float* cosv, float* sinv, int tokens, int naxes, const int* axes_dim, float theta,
                   cudaStream_t st);

// ---- pointwise.cu
int mdb_act_fwd(const void* x, void* y, const void* bias, long long n, int cols, int act, cudaStream_t st);
int mdb_act_bwd(const void* x, const void* dy, void* dx, const void* bias, long long n, int cols, int act,
                cudaStream_t st);
int mdb_glu_fwd(const void* x, void* y, long long rows, int F, int ldx, int ldy, int act, int second, cudaStream_t st);
int mdb_glu_bwd(const void* x, const void* dy, void* dx, long long rows, int F, int ldx, int lddy, int lddx, int act,
                int second, cudaStream_t st);
int mdb_act_strided(const void* x, long long ldx, const void* dy, long long lddy, void* out, long long ldo,
                    long long rows, int cols, int act, cudaStream_t st);
int mdb_gate_residual(const void* x, const void* y, const void* gate, void* out, long long rows, int D,
                      int gate_stride, int rows_per_group, int tanh_gate, cudaStream_t st);
int mdb_cfg_euler(float* x, const void* vc, const void* vu, void* x_bf16, long long n, float dt, float s, int mode,
                  cudaStream_t st);
int mdb_flow_match(const float* x0, const float* eps, const float* sigma, void* xt, float* target, long long n,
                   long long per_sample, cudaStream_t st);
int mdb_mse_loss(const void* pred, const float* target, void* grad, float* loss_sum, long long n, float grad_coef,
                 cudaStream_t st);
int mdb_randn(float* out_f32, void* out_bf16, long long n, unsigned long long seed, unsigned long long offset,
              cudaStream_t st);
int mdb_fp8_quant_rows(const void* x, void* q, float* scale, long long rows, int D, int ldx, int ldq, cudaStream_t st);
// MXFP8 GEMM operands: E4M3 bytes [rows, K] plus scale chunks [ceil(rows/128)][K/128][512] in the tensor core's layout
// (byte (row % 32) * 16 + (row % 128 / 32) * 4 + k32 % 4); scale buffers are padded to whole tiles and preset to 127
int mdb_mxfp8_quant_rows(const void* x, void* q, void* sf, long long rows, int K, long long ldx, cudaStream_t st);
int mdb_gemm_mxfp8(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* out, const void* bias, int M, int N,
                   int K, int ld_out, int* status, cudaStream_t st);
// MX formats: 32-element blocks with one E8M0 scale byte; fp4 != 0: E2M1 nibbles (16 bytes per block), else E4M3 bytes
int mdb_mx_dequant(const void* q, const void* scales, void* y, long long n_blocks, int fp4, cudaStream_t st);
int mdb_mx_quant(const void* x, void* q, void* scales, long long n_blocks, int fp4, cudaStream_t st);
int mdb_fp8_dequant(const void* q, const float* row_scale, float tensor_scale, void* y, long long rows, int D,
                    cudaStream_t st);

// ---- conv_norm.cu (NHWC)
// scratch: mdb_group_norm_scratch_floats(N, HW, C, G, wgrad) fp32 values (wgrad < 0: forward; 0 / 1: backward without / with dw, db)
long long mdb_group_norm_scratch_floats(int N, int HW, int C, int G, int wgrad);
int mdb_group_norm_bwd(const void* x, const void* dy, void* dx, float* scratch, const void* w, const void* b, float* dw, float* db,
                       int N, int HW, int C, int G, float eps, int act, cudaStream_t st);
// stats: scratch of mdb_group_norm_scratch_floats(N, HW, C, G, -1) fp32 values; its first 2 * N * G hold (mean, rstd) afterwards
int mdb_group_norm(const void* x, void* y, float* stats, const void* w, const void* b, int N, int HW, int C, int G,
                   float eps, int act, cudaStream_t st);
int mdb_upsample2x(const void* x, void* y, int N, int H, int W, int C, cudaStream_t st);
int mdb_avgpool2x(const void* x, void* y, int N, int H, int W, int C, cudaStream_t st);

// GroupNorm (+ optional SiLU) that brings its own workspace. This entry point has no counterpart in the reference
// project; it exists for hosts that must not allocate while they run:
//   * a C/C++ or ctypes host that drives these kernels without a tensor library, so there is no caching allocator
//     to ask for the small per-(sample, group) statistics buffer that mdb_group_norm needs;
//   * a serving process that sized all of its device memory up front and wants a call that cannot fail, fragment
//     or synchronise the device by asking the CUDA allocator for more.
// The (mean, rstd) pairs live in a fixed array inside the library's device image:
// MDB_GROUP_NORM_STATIC_MAX_GROUPS pairs (64 KiB) per device. N * G beyond that is refused with
// MDB_ERR_STATIC_WS_TOO_SMALL and a line on stderr; nothing is launched in that case.
// The call itself never calls cudaMalloc, cudaFree or any routine that allocates.
// What the caller has to know:
//   * The first call on each device looks up the array's address (and may make the driver load the module). Make that
//     first call once, on an ordinary stream, before starting any stream capture.
//   * Every call on a device uses the same array. Calls that overlap in time (two streams, two host threads) race on
//     it and give wrong results; order them on one stream or with events.
//   * Nothing in the array has to start at zero: each call first writes every pair that it later reads, so whatever an
//     earlier call left behind is never seen.
// x, y: bf16 NHWC [N, H*W, C]; w, b: bf16 [C] or NULL; C % 8 == 0 and C % G == 0; act: 0 none, 2 SiLU (the activation codes used across this library).
// Returns 0, a negative argument error, or a positive cudaError_t value.
#define MDB_GROUP_NORM_STATIC_MAX_GROUPS 8192
#define MDB_ERR_STATIC_WS_TOO_SMALL (-20)
int mdb_group_norm_static_ws(const void* x, void* y, const void* w, const void* b, int N, int HW, int C, int G,
                             float eps, int act, cudaStream_t st);

// ---- optim.cu
int mdb_lion_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems, int p_bf16, int g_bf16,
                   float lr, float beta1, float beta2, float wd, float grad_scale, const int* status, cudaStream_t st);
int mdb_stable_adamw_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems, int p_bf16,
                           int g_bf16, float lr, float beta1h, float beta2h, float eps, float wd, float grad_scale,
                           float* rms_acc, const int* status, cudaStream_t st);
int mdb_adamw_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems, int p_bf16,
                    int g_bf16, int m_bf16, float lr, float beta1, float beta2, float eps, float wd, int step,
                    float grad_scale, const float* norm_sq, float max_norm, unsigned int seed, int stochastic,
                    const int* status, cudaStream_t st);   // status (may be NULL): device status word; not OK -> no update
int mdb_sumsq_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems, int g_bf16,
                    float* out, cudaStream_t st);
int mdb_ema_multi(const MdbTensorEntry* tensors, const int* chunks, int num_chunks, int chunk_elems, int p_bf16,
                  float decay, cudaStream_t st);

// AdamW with block-wise (256 elements) 8-bit moments: qm / qv hold code-book indices, am / av one fp32 maximum per
// block; code_s / code_u are the 256-entry signed / unsigned code books (ascending). step == 1 starts from zero moments.
int mdb_adamw8bit(void* p, const void* g, void* qm, void* qv, float* am, float* av, const float* code_s,
                  const float* code_u, long long n, int p_bf16, int g_bf16, float lr, float b1, float b2, float eps,
                  float wd, int step, float grad_scale, cudaStream_t st);

// ---- attention_tcgen05.cu
// q,k,v,o: bf16 with element strides (batch, seq, head); head_dim contiguous (Dh = 128 or 64).
// lse: optional fp32 [B, H, Sq] (natural-log-sum-exp of the scaled scores) for the backward pass.
// kv_len: optional int32 [B] number of valid keys per batch entry (key padding mask).
typedef struct MdbAttnArgs {
  const void* q; const void* k; const void* v; void* o;
  float* lse;
  const int* kv_len;
  int B, H, Sq, Skv, Dh;
  long long q_strides[3], k_strides[3], v_strides[3], o_strides[3];  // (batch, seq, head) in elements
  float scale;
  int num_sms;
  int* status;
  // Peer-routed output (route_rows_a > 0): query row t < route_split belongs to rank t / route_rows_a and is stored
  // at row t % route_rows_a of o_route_a[rank]; row t >= route_split belongs to rank (t - route_split) / route_rows_b
  // and goes to o_route_b[rank]. Each table entry already points at this rank's head block inside the owner's
  // buffer; o_strides then describe the OWNER's buffer. This is the inverse Ulysses all-to-all done by the
  // attention kernel's own epilogue.
  void* o_route_a[8];
  void* o_route_b[8];
  int route_rows_a, route_split, route_rows_b;
} MdbAttnArgs;
int mdb_attention_fwd(const MdbAttnArgs* a, cudaStream_t st);
// debugging aid: per-kv-tile clock64 time line of CTA (0,0,0) of the following forward launches ([4][len] int64; NULL: off)
void mdb_attention_set_trace(long long* trace, int len);

// ---- shader_filters.cu: RGBA fp32 image filters (op codes and parameter layout documented at the definition)
int mdb_image_filter(int op, const float* in, float* out, float* tmp, int H, int W, const float* params, int nparams,
                     const void* aux, cudaStream_t st);

// ---- attention_bwd_tcgen05.cu
// delta: fp32 workspace [B, H, Sq] filled by the call (rowsum(dO o O)); lse from the forward.
typedef struct MdbAttnBwdArgs {
  const void* q; const void* k; const void* v; const void* o; const void* dout;
  void* dq; void* dk; void* dv;
  const float* lse;
  float* delta;
  const int* kv_len;
  int B, H, Sq, Skv, Dh;
  long long q_strides[3], k_strides[3], v_strides[3], o_strides[3], do_strides[3];
  long long dq_strides[3], dk_strides[3], dv_strides[3];
  float scale;
  int* status;
} MdbAttnBwdArgs;
int mdb_attention_bwd(const MdbAttnBwdArgs* a, cudaStream_t st);

#ifdef __cplusplus
}
#endif
