/*
 * Multi-GPU helpers of the quantised-matmul path: how a problem is cut over the GPUs of one box, and the optional gather of the
 * output shards. One process per GPU; nothing here is needed for the matmuls themselves, which run on shards with no
 * collective on the data path.
 *
 * The reference has no multi-device code for these operators (its aclnn entry points see one device), so nothing below
 * replaces a reference interface. The alignment arguments come from its data formats: INT4 weights are packed eight per
 * INT32 along n (matmul/weight_quant_batch_matmul_v2/op_host/op_api/aclnn_weight_quant_batch_matmul_v2.cpp:1482-1524) and
 * per-block weight scales cover 128 columns (matmul/quant_batch_matmul_v3/op_api/quant_matmul_checker.cpp:724-767).
 *
 * NCCL is resolved at run time from the libnccl.so.2 already in the process (or on the loader path); without it the
 * communicator functions return cudaErrorNotSupported and the rest of the library is unaffected.
 */
#ifndef OPSNN_B200_SHARD_H_
#define OPSNN_B200_SHARD_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OPSNN_SHARD_API __attribute__((visibility("default")))

/* [begin, end) of `rank`'s share of `total` items cut into `world` contiguous parts whose boundaries are multiples of
 * `multiple` (8 for INT4 weight columns, 128 for per-block weight columns, 512 to keep whole decode strips, 1 for batches).
 * Units of `multiple` are dealt as evenly as possible, the first ranks taking the extra ones; a ragged tail shorter than
 * `multiple` goes to the last rank that owns anything. Pure host arithmetic. */
OPSNN_SHARD_API void opsnn_shard_range(int64_t total, int32_t world, int32_t rank, int64_t multiple, int64_t* begin, int64_t* end);

/* A communicator over the ranks of one box. Rank 0 calls opsnn_comm_unique_id and hands the 128 bytes to the other ranks by
 * whatever means the host has; every rank then calls opsnn_comm_init with its device current. */
OPSNN_SHARD_API int32_t opsnn_comm_unique_id(void* id128);
OPSNN_SHARD_API int32_t opsnn_comm_init(const void* id128, int32_t world, int32_t rank, void** comm);
OPSNN_SHARD_API int32_t opsnn_comm_destroy(void* comm);

/* Column shards -> the whole (m, n_total) row-major output on every rank. y_local is this rank's (m, width) shard with
 * y_local_ld elements per row, width = its opsnn_shard_range(n_total, world, rank, multiple); elem_bytes is 1, 2 or 4.
 * Enqueues one strided copy, one ncclAllGather and one interleave kernel on `stream`; workspace per
 * opsnn_gather_columns_workspace. */
OPSNN_SHARD_API uint64_t opsnn_gather_columns_workspace(int32_t world, int64_t m, int64_t n_total, int64_t multiple, int32_t elem_bytes);
OPSNN_SHARD_API int32_t opsnn_gather_columns(void* comm, const void* y_local, int64_t y_local_ld, int64_t m, int64_t n_total, int64_t multiple,
                                             int32_t elem_bytes, void* y_full, void* workspace, uint64_t workspace_size, void* stream);

/* Batch shards (equal shares, batch_total % world == 0) -> the whole output on every rank: one ncclAllGather, in place
 * when y_local already is this rank's slot of y_full. */
OPSNN_SHARD_API int32_t opsnn_gather_batch(void* comm, const void* y_local, int64_t batch_total, uint64_t bytes_per_batch, void* y_full, void* stream);

/* ---- the gather folded into the decode kernels' epilogue (column shards, at most 8 ranks of one node) ----------------------
 * For the small outputs of the decode regime (m <= 16) a separate all-gather costs more than the matmul (tens of microseconds of
 * launch and NCCL latency for ~100 KB per rank). Instead every rank holds the full (m, n_total) output in memory that all ranks
 * have mapped (CUDA IPC), and the streaming decode kernels store every element of their shard straight into every rank's copy -
 * plain stores over NVLink from the epilogue, no TMA from or multicast into peer memory. opsnn_comm_arrive_and_wait then
 * tells the other ranks that this rank's stores are done and waits until theirs are: one single-warp kernel, a release store per
 * peer and a bounded poll per peer (about a second; a wait that runs out sets the word opsnn_comm_status reads, the kernel
 * returns, nothing hangs).
 *
 *   opsnn_comm_symmetric_alloc   collective; `bytes` of zeroed device memory on every rank; peers (optional, [world]) receives
 *                                every rank's block as mapped into this process, peers[rank] == *local.
 *   opsnn_comm_bind_columns      registers y_local (this rank's (m, width) shard, the y of the calls to come) as a column shard of
 *                                y_full_local (a symmetric allocation, (m, n_total) row-major, same element type). From then on
 *                                aclnnWeightQuantBatchMatmulV2 / V3 / opsnn_wqbmm_launch calls whose y is y_local and that run on a
 *                                streaming decode kernel write y_local and every rank's full output; a bound call that would run
 *                                on another kernel is refused (cudaErrorNotSupported) rather than silently left ungathered.
 *   opsnn_comm_arrive_and_wait   collective on `stream`, after the bound call: afterwards every rank's full output is complete.
 *   opsnn_comm_allgather_columns the other way round, for any producer of y_local: ONE kernel of `world` CTAs after it copies the
 *                                rank's (m, width) shard into every rank's full output with 16-byte peer stores (rows are
 *                                contiguous on both sides), announces and awaits arrival like opsnn_comm_arrive_and_wait. With
 *                                many ranks this beats the epilogue form (whose peer stores are 2-byte and scattered by the MMA
 *                                fragment layout): 8 GPUs, 16 x 3584 shards. No binding is involved.
 * No counterpart in the reference (it has no multi-device code for these operators). */
OPSNN_SHARD_API int32_t opsnn_comm_symmetric_alloc(void* comm, uint64_t bytes, void** local, void** peers);
OPSNN_SHARD_API int32_t opsnn_comm_symmetric_free(void* comm, void* local);
OPSNN_SHARD_API int32_t opsnn_comm_bind_columns(void* comm, const void* y_local, const void* y_full_local, int64_t n_total, int64_t multiple);
OPSNN_SHARD_API int32_t opsnn_comm_unbind(const void* y_local);
OPSNN_SHARD_API int32_t opsnn_comm_arrive_and_wait(void* comm, void* stream);
OPSNN_SHARD_API int32_t opsnn_comm_allgather_columns(void* comm, const void* y_local, int64_t y_local_ld, int64_t m, const void* y_full_local,
                                                     int64_t n_total, int64_t multiple, int32_t elem_bytes, void* stream);
OPSNN_SHARD_API uint32_t opsnn_comm_status(void* comm, int32_t reset);

#ifdef __cplusplus
}
#endif
#endif /* OPSNN_B200_SHARD_H_ */
