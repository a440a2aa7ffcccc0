// C interface of the peer-memory communication kernels (comm_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MDB_MAX_RANKS 8
#define MDB_FLAG_SLOTS 8

#ifdef __cplusplus
extern "C" {
#endif

// device-visible addresses of the same symmetric buffer on every rank (index = rank)
typedef struct MdbPeerTable {
  void* p[MDB_MAX_RANKS];
} MdbPeerTable;

// flags buffers: int32 [slots][MDB_MAX_RANKS] per rank, monotonic epochs
// value > 0: explicit epoch. value == 0: epoch from device counters (int[2 * MDB_FLAG_SLOTS], local, zero-initialised)
int mdb_flag_signal(const MdbPeerTable* flags, int slot, int rank, int world, int value, int* counters,
                    cudaStream_t st);
int mdb_flag_wait(const int* my_flags, int slot, int world, int value, int* counters, int* status, cudaStream_t st);

// signal + wait in one launch
int mdb_flag_barrier(const MdbPeerTable* flags, const int* my_flags, int slot, int rank, int world, int value, int* counters,
                     int* status, cudaStream_t st);
// staged reduce-scatter tail: barrier on `slot` (explicit epoch > 0), then out = residual + gate * (sum of the `world`
// bf16 slots of stage[world][rows][D] + bias). bias / residual / gate may be NULL. Exactly one of out (bf16 [rows, D]) and
// accum (fp32 [rows, D], += the result: gradient accumulation) is given.
// reduce-scatter tail + AdamW on the owner's shard in one launch (stage: bf16 [world][n]); see rs_adamw_kernel
int mdb_rs_adamw(const MdbPeerTable* flags, const int* my_flags, int slot, int epoch, int rank, int world, const void* stage, long long n,
                 float* master, float* m, float* v, void* shadow, float lr, float beta1, float beta2, float eps, float wd, int step,
                 float grad_scale, int* status, cudaStream_t st);
int mdb_rs_finalize(const MdbPeerTable* flags, const int* my_flags, int slot, int epoch, int rank, int world,
                    const void* stage, long long rows, int D, const void* bias, const void* residual, const void* gate,
                    int rows_per_group, long long gate_stride, void* out, float* accum, int* status, cudaStream_t st);

// all-gather by peer loads into dst = [world][chunk_bytes]
int mdb_peer_gather(const MdbPeerTable* src, void* dst, long long chunk_bytes, int rank, int world, int copy_local,
                    cudaStream_t st);

int mdb_dp_reduce_shard(const MdbPeerTable* grads, const void* grads_mc, const int* my_flags, int ready_slot, int epoch,
                        int world, long long lo, long long hi, float* red, float* sumsq, int* status, cudaStream_t st);
// status (may be NULL): when the device's status word is not OK the rank publishes NaN, which makes every peer skip its update
int mdb_publish_scalar(const MdbPeerTable* scalars, const MdbPeerTable* flags, const float* value, int slot, int rank,
                       int world, int epoch, const int* status, cudaStream_t st);
int mdb_dp_adamw_shard(const MdbPeerTable* params, void* params_mc, const MdbPeerTable* flags, const int* my_flags,
                       const float* my_scalars, int norm_slot, int done_slot, int epoch, int rank, int world,
                       long long lo, long long hi, const float* red, float* m, float* v, float lr, float beta1,
                       float beta2, float eps, float wd, int step, float grad_scale, float max_norm, float* norm_out,
                       int* done_counter, int* status, cudaStream_t st);

// Wall-clock limit (nanoseconds) of every bounded device-side wait, per translation unit; one second by default. Applies to
// the current device.
int mdb_set_wait_limit_gemm(unsigned long long ns);
int mdb_set_wait_limit_attn_fwd(unsigned long long ns);
int mdb_set_wait_limit_attn_bwd(unsigned long long ns);
int mdb_set_wait_limit_comm(unsigned long long ns);
int mdb_set_wait_limit_mxfp8(unsigned long long ns);

#ifdef __cplusplus
}
#endif
