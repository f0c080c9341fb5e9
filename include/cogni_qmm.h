/*
 * cogni_qmm — C ABI of the B200 (sm_100a) quantized-matmul engine for GGUF weights.
 *
 * This is the boundary a host runtime binds through its FFI.  Every entry point takes
 * plain pointers and sizes; device pointers are ordinary CUDA device addresses (the same
 * 64-bit value the Driver API calls CUdeviceptr), `stream` is a CUstream / cudaStream_t
 * (NULL = the default stream).  Calls run in whatever CUDA context is current on the
 * calling thread (a context made with cuCtxCreate or the primary context both work).
 *
 * Return value: 0 on success.  Values 1..999 are CUDA error codes (cudaError_t, numerically
 * equal to the Driver API's CUresult for the errors a launch can raise), values >= 1000 are
 * the COGNI_QMM_ERR_* codes below.  cogni_qmm_status_string() names either kind.
 * The reference's convention is "every driver call returns Int32, non-zero raises"
 * (src/ml/cuda/driver.cr:57-59); a binding wraps each call in the same check!.
 *
 * Weights are always the raw GGUF block bytes, row-major [out_dim rows][in_dim/block
 * blocks], exactly as GGUFFile#read_tensor_raw returns them (src/ml/gguf/reader.cr:169-194);
 * nothing is repacked on the host.
 */
#ifndef COGNI_QMM_H
#define COGNI_QMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COGNI_QMM_ABI_VERSION 1

/* ggml tensor type ids, identical to ML::GGUF::TensorType (src/ml/gguf/reader.cr:36-50). */
#define COGNI_QMM_TYPE_Q8_0 8
#define COGNI_QMM_TYPE_Q4_K 12
#define COGNI_QMM_TYPE_Q5_K 13
#define COGNI_QMM_TYPE_Q6_K 14
#define COGNI_QMM_TYPE_IQ4_NL 20

#define COGNI_QMM_OK 0
#define COGNI_QMM_ERR_TYPE 1001      /* tensor type not supported by this engine           */
#define COGNI_QMM_ERR_ARG 1002       /* null pointer, non-positive size, in_dim not a block multiple */
#define COGNI_QMM_ERR_ALIGN 1003     /* a device pointer is not aligned as documented      */
#define COGNI_QMM_ERR_SCRATCH 1004   /* scratch buffer too small                           */
#define COGNI_QMM_ERR_DEVICE 1005    /* device is not compute capability 10.x             */
#define COGNI_QMM_ERR_LIMIT 1006     /* size beyond a documented fixed maximum             */
#define COGNI_QMM_ERR_TIMEOUT 1007   /* a bounded device-side wait expired (results invalid) */
#define COGNI_QMM_ERR_NCCL_MISSING 1008 /* libnccl.so.2 could not be loaded                    */
#define COGNI_QMM_ERR_NCCL_BASE 2000 /* 2000 + ncclResult_t of a failed NCCL call           */

/* Output element types of the prefill GEMM. */
#define COGNI_QMM_OUT_F32 0
#define COGNI_QMM_OUT_BF16 1

/* ABI version of the loaded library (== COGNI_QMM_ABI_VERSION it was built with). */
int cogni_qmm_abi_version(void);

/* Human-readable name of a status returned by any entry point. Never NULL. */
const char *cogni_qmm_status_string(int status);

/*
 * Bounded waits.  Every device-side wait of the tiled kernels (on a copy, a stage, a counter) has
 * a wall-clock limit of one second; a wait that runs out is counted, the kernel carries on to its
 * end with invalid results, and from then on every wait of every launch gives up at once, so a
 * broken pipeline can never hang the GPU.  (No counterpart in the reference, whose kernels do not
 * wait on anything.)
 *   cogni_qmm_wait_timeouts        how many waits have expired since the library was loaded or the
 *                                  counters were last reset; 0 in a healthy process.  Synchronises
 *                                  the device.  cogni_qmm_matmul_add_host checks it itself and
 *                                  returns COGNI_QMM_ERR_TIMEOUT.
 *   cogni_qmm_reset_wait_timeouts  clears the counters and the kernels' cross-CTA tickets after the
 *                                  host has dealt with an expiry; launches are valid again.
 *                                  Synchronises the device.
 */
unsigned cogni_qmm_wait_timeouts(void);
int cogni_qmm_reset_wait_timeouts(void);

/* Block geometry: TensorType#block_bytes / #block_elements (reader.cr:53-80).
 * Return -1 for a type this engine does not handle. */
int cogni_qmm_block_bytes(int type);
int cogni_qmm_block_elements(int type);

/* Bytes of one weight row / of a whole [out_dim, in_dim] tensor: the row_bytes the
 * reference computes in every matmul_add_* (quant_matmul.cr:46-48) and
 * TensorInfo#data_bytes (reader.cr:119-127). -1 on a bad type or in_dim. */
int64_t cogni_qmm_row_bytes(int type, int in_dim);
int64_t cogni_qmm_tensor_bytes(int type, int out_dim, int in_dim);

/*
 * Bulk dequantisation on the device: replaces Dequant.dequantize for Q8_0 / Q4_K / Q5_K /
 * Q6_K (src/ml/gguf/dequant.cr:20-32, 53-71, 106-142, 146-193, 197-236).  All arithmetic
 * is f32 in the reference's operation order, so the result is bit-identical to the CPU
 * dequantiser.  d_w: raw blocks (2-byte aligned is enough), d_out: n_elements floats.
 * n_elements must be a multiple of the block size.
 */
int cogni_qmm_dequantize(int type, const void *d_w, int64_t n_elements, float *d_out,
                         void *stream);

/*
 * Decode GEMV, batch 1..16 rows of x against one quantized weight matrix:
 *     y[b, o] = addend[b*addend_stride + o] + sum_j x[b, j] * dequant(W[o, j])
 * Replaces QuantMatmul.matmul_add on the device (src/ml/gguf/quant_matmul.cr:20-36, with
 * bias as the accumulator start) and the reference's GEMV kernels
 * q4_k_gemv_warp4_f32 / _add_ / _batched / _tbatch4 and their Q5_K / Q6_K / Q8_0 twins
 * (src/ml/cuda/kernels/q4k_gemv_probe.ptx:219,437,1362,1584; q5k_gemv_probe.ptx:5,237,589;
 * q6k_gemv_probe.ptx:193,398,609,977,1582; bin/cuda_q8_gemv_probe.cr:126).
 *   d_w       raw GGUF blocks, [out_dim][in_dim], 16-byte aligned base
 *   d_x       f32 [batch, in_dim] row-major
 *   d_addend  NULL, or f32: addend_stride == 0 -> a bias of out_dim entries added to every
 *             batch row (matmul_add's bias); addend_stride == out_dim -> a residual
 *             [batch, out_dim] (the *_gemv_add_* kernels). May alias d_y.
 *   d_y       f32 [batch, out_dim]
 * The weight bytes are streamed from HBM once per call whatever the batch.  Accumulation is
 * fp32.  batch > 16 is processed in groups of 16.
 */
int cogni_qmm_gemv(int type, const void *d_w, const float *d_x, const float *d_addend,
                   int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                   void *stream);

/*
 * cogni_qmm_gemv for weights that are resident: identical arguments and result, with one extra
 * promise from the caller — the weight bytes at d_w were complete before the kernel that precedes
 * this call in `stream` was launched.  That is the reference's runner lifecycle (upload_weights
 * once, then run_sequence many times; src/ml/cuda/qwen_recurrent_layer_runner.cr:570-587,
 * 1158-1266).  The kernel may then start fetching weights while the preceding kernel of the
 * stream is still draining (programmatic dependent launch); x, the addend and y are still only
 * touched after the preceding kernel has completed.
 */
int cogni_qmm_gemv_resident(int type, const void *d_w, const float *d_x, const float *d_addend,
                            int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                            void *stream);

/*
 * cogni_qmm_gemv_many with the RMSNorm of the hidden state fused into the activation pass:
 *     xn[b, k] = x[b, k] * (1 / sqrt(mean_k(x[b, k]^2) + eps)) * norm_weight[k]
 *     y_j[b, o] = addend_j[b*addend_stride + o] + sum_k xn[b, k] * dequant(W_j[o, k])
 * the sum of squares in f64, the two products in f32 from left to right, as Qwen35CPU#rms_norm
 * does (src/ml/gguf/qwen35_cpu.cr:484-490), followed by qmatvec_many (qwen35_cpu.cr:1793, 1883:
 * attn_norm -> qkv / gate / alpha / beta, post_attention_norm -> ffn_gate / ffn_up); replaces the
 * reference's add_rmsnorm / rmsnorm probe kernels (deltanet_step_probe.ptx:1324) plus the GEMVs.
 * Where the tiled kernel takes the shapes (in_dim a multiple of 256, at most 32
 * matrices) xn is never written; otherwise it goes to d_x_scratch (f32 [batch, in_dim],
 * COGNI_QMM_ERR_SCRATCH if NULL) and cogni_qmm_gemv_many runs on that.  norm_weight: f32 [in_dim]
 * on the device, 16-byte aligned.  Other arguments as cogni_qmm_gemv_many.
 */
int cogni_qmm_gemv_many_rmsnorm(int type, int n_weights, const void *const *d_w, const float *d_x,
                                const float *d_norm_weight, float eps,
                                const float *const *d_addend, int64_t addend_stride,
                                float *const *d_y, const int *out_dims, float *d_x_scratch,
                                int in_dim, int batch, int resident, void *stream);

/*
 * Token-embedding gather from the quantized table (one of the steps next to the matmul path):
 *     out[t, :] = dequant(row d_token_ids[t] of the [vocab, n_embd] table),  f32 [n_tokens, n_embd]
 * bit-identical to Dequant.dequantize of that row, as Qwen35CPU#embedding_lookup does
 * (src/ml/gguf/qwen35_cpu.cr:3305-3332); replaces embed_q4k_f32_from_token_id_cuda
 * (src/ml/cuda/kernels/embed_q4k_probe.ptx:5) and the Metal embedding_q4k/q6k_from_token_id
 * (src/ml/gguf/qwen35_metal.cr:848-900) for all four types.  d_token_ids is a device array of
 * int32, e.g. the top_index written by cogni_qmm_gemv_top1, so that argmax -> next embedding stays
 * on the device.  The reference raises for an id outside [0, vocab); here such a row is filled with
 * zeros and, if d_status is not NULL, *d_status (device int32, zeroed by the caller) is raised to
 * 1 + the index of such a token.  n_embd must be a multiple of the block size.
 */
int cogni_qmm_embedding_lookup(int type, const void *d_table, int vocab, int n_embd,
                               const int32_t *d_token_ids, int n_tokens, float *d_out,
                               int32_t *d_status, void *stream);

/*
 * cogni_qmm_gemv_top1 with the output RMSNorm fused in: the argmax of W (RMSNorm(x) * norm_weight)
 * per row, the norm as in cogni_qmm_gemv_many_rmsnorm.  This is the reference's
 * rmsnorm_project_top1_rows (src/ml/gguf/qwen35_metal.cr:9187) and the CUDA head runner's
 * rmsnorm -> lm_head -> top-1 chain (src/ml/cuda/qwen_output_head_runner.cr:884-947) as one launch
 * where the tiled kernel takes the shape (in_dim a multiple of 256); otherwise the
 * normalised rows go to d_x_scratch (f32 [batch, in_dim], COGNI_QMM_ERR_SCRATCH if NULL) first.
 * d_scratch / scratch_bytes as for cogni_qmm_gemv_top1.
 */
int cogni_qmm_gemv_top1_rmsnorm(int type, const void *d_w, const float *d_x,
                                const float *d_norm_weight, float eps, int in_dim, int out_dim,
                                int batch, int32_t index_base, void *d_scratch, size_t scratch_bytes,
                                float *d_x_scratch, int32_t *d_top_index, float *d_top_value,
                                int64_t *d_top_key, int resident, void *stream);

/*
 * lm_head with the two best tokens per row (the verifier's top-1 / top-2 and their margin):
 * the logits of all `batch` rows go to the scratch buffer with the GEMV of this engine, one more
 * launch scans them and leaves, for row b, d_top_index[2b], d_top_value[2b] (the argmax, same tie
 * rule as cogni_qmm_gemv_top1) and d_top_index[2b+1], d_top_value[2b+1] (the runner-up); d_top_key
 * (optional, 2 * batch int64) receives the packed keys for a cross-shard merge (the two largest
 * keys over all shards are the global answer).  Replaces the logits GEMV followed by
 * output_top2_partial_scan_probe / output_top2_partial_reduce_probe
 * (src/ml/cuda/qwen_output_head_runner.cr:158-338, 864-904).  out_dim >= 2.  The scratch buffer
 * (cogni_qmm_gemv_top2_scratch_bytes, 8-byte aligned) must be zero-filled once before its first
 * use; the logits stay readable in it after the call, f32 [batch, out_dim] at its end.
 */
size_t cogni_qmm_gemv_top2_scratch_bytes(int out_dim, int batch);
int cogni_qmm_gemv_top2(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                        int batch, int32_t index_base, void *d_scratch, size_t scratch_bytes,
                        int32_t *d_top_index, float *d_top_value, int64_t *d_top_key, int resident,
                        void *stream);

/*
 * The FFN down projection with the SwiGLU product fused into its activation pass:
 *     y[b, o] = addend[b*addend_stride + o] + sum_k (silu(gate[b, k]) * up[b, k]) * dequant(W[o, k])
 * with silu(v) = v / (1 + exp(-v)) in f32 (src/ml/gguf/qwen35_cpu.cr:512-519, 1716-1718; the
 * reference's swiglu_probe kernel, src/ml/cuda/kernels/deltanet_step_probe.ptx:1076, followed by
 * the down-projection GEMV).  gate and up are f32 [batch, in_dim] device buffers, 16-byte aligned.
 * Where the tiled kernel takes the shape (in_dim a multiple of 256) the product is
 * formed while the activations are quantised and never written to memory; otherwise it is
 * written to d_x_scratch (f32 [batch, in_dim], COGNI_QMM_ERR_SCRATCH if NULL) and the plain GEMV
 * runs on that.  `resident` as in cogni_qmm_gemv_resident.
 */
int cogni_qmm_gemv_swiglu(int type, const void *d_w, const float *d_gate, const float *d_up,
                          const float *d_addend, int64_t addend_stride, float *d_y,
                          float *d_x_scratch, int in_dim, int out_dim, int batch, int resident,
                          void *stream);

/*
 * Several weight matrices of one type and in_dim against the SAME x in one launch:
 *     y_j[b, o] = addend_j[b*addend_stride + o] + sum_k x[b, k] * dequant(W_j[o, k])
 * Replaces Qwen35CPU.qmatvec_many (src/ml/gguf/qwen35_cpu.cr:1419-1490: qkv / gate / alpha / beta
 * from one hidden state, ffn_gate + ffn_up) and the dual GEMV kernel
 * (src/ml/cuda/kernels/q4k_dual_gemv_probe.ptx:5).  The matrices' row tiles form one work
 * sequence, so the launch ramp and tail are paid once and the rows balance over the SMs together.
 *   d_w, d_y, out_dims   HOST arrays of n_weights device pointers / row counts
 *   d_addend             NULL, or a HOST array of n_weights device pointers (entries may be NULL)
 *   resident             non-zero: the promise of cogni_qmm_gemv_resident for every matrix
 * Other arguments as for cogni_qmm_gemv.  batch > 2 or unaligned pointers run one GEMV per matrix.
 */
int cogni_qmm_gemv_many(int type, int n_weights, const void *const *d_w, const float *d_x,
                        const float *const *d_addend, int64_t addend_stride, float *const *d_y,
                        const int *out_dims, int in_dim, int batch, int resident, void *stream);

/*
 * Row-sharded decode over the GPUs of one box with the exchange fused into the GEMV launch.
 * (No counterpart in the reference, which is single-GPU; the partition is the one its layout
 * suggests: output rows are independent and stored back to back, src/ml/gguf/qwen35_weights.cr:209-212.)
 *
 * Every rank holds the rows [rank * N / G, (rank + 1) * N / G) of each matrix and a gather buffer
 * laid out identically on all ranks: [batch][N] WORDS of 8 bytes, (f32 value, u32 epoch).  d_y[j]
 * points INTO this rank's buffer at the word of its first row (column rank * N / G of batch row 0),
 * y_pitch = N.  The kernel writes every output value as one 8-byte store (value, epoch) there and,
 * with ordinary stores over NVLink, at the same place of every peer's buffer (peer-mapped memory:
 * cuIpcOpenMemHandle / cuMemMap by the host).  Value and epoch arrive together, so there is no
 * fence, no flag and no barrier: a later launch whose activations are such a buffer passes
 * wait_previous = 1 and polls every word it reads until it carries the epoch of the exchange
 * before it (a bounded wait, cogni_qmm_wait_timeouts).  No NCCL call, no extra launch, no
 * multicast load.
 *
 *   world, rank     ranks of the box (world <= 8) and this one
 *   peer_offset[g]  BYTES from an address in this rank's gather buffer to the same place in rank
 *                   g's buffer as mapped into this process (entry [rank] is ignored)
 *   epoch, ticket   two device words of this rank, zero-initialised before the first exchange:
 *                   the count of exchanges this rank has completed, and the arrivals of the
 *                   running launch
 * All ranks must issue the same sequence of exchanging launches on one exchange (epoch / ticket
 * pair).  wait_previous = 1 means: d_x is the gather buffer written by the exchanging launch
 * issued immediately before this one on the same exchange (in_dim = its N).  A buffer may be
 * rewritten by the launch after next: two buffers alternating are enough for a chain.  Shapes the
 * tiled kernel does not take in one launch (batch > 8, in_dim not a multiple of 256, ...) return
 * COGNI_QMM_ERR_LIMIT: run cogni_qmm_gemv_many and an all-gather instead.
 * cogni_qmm_exchange_unpack strips the epochs for a reader that is not a GEMV of this library:
 * out[i] = value of word i, after waiting (bounded) until the word carries `epoch`.
 */
typedef struct cogni_qmm_exchange {
  int32_t world, rank;
  int64_t peer_offset[8];
  uint32_t *epoch;
  uint32_t *ticket;
} cogni_qmm_exchange;

int cogni_qmm_gemv_many_exchange(int type, int n_weights, const void *const *d_w, const float *d_x,
                                 const float *const *d_addend, int64_t addend_stride,
                                 float *const *d_y, int64_t y_pitch, const int *out_dims, int in_dim,
                                 int batch, int resident, const cogni_qmm_exchange *exchange,
                                 int wait_previous, void *stream);
int cogni_qmm_exchange_unpack(const void *d_words, int64_t n, uint32_t epoch, float *d_out,
                              void *stream);

/*
 * The same two sharded operations with NCCL as the exchange step, on a communicator the host owns
 * (ncclCommInitRank / ncclCommInitAll in the host's binding; this library neither creates nor
 * destroys communicators).  (No counterpart in the reference, which has no collective call.)
 *
 * cogni_qmm_sharded_gemv_nccl: rank's row shard (rows = N / world rows of the matrix) against the
 * replicated x, written into block `rank` of d_gather ([world][batch][rows] f32), then one
 * in-place ncclAllGather: every rank ends with all blocks.
 *
 * cogni_qmm_sharded_top1_nccl: the fused lm_head on rank's vocabulary shard (index_base = its first
 * row), then ncclAllReduce(ncclMax) on the int64 keys (highest value, lowest index: the tie rule of
 * cogni_qmm_gemv_top1) and the unpacking of the winning keys: d_top_index / d_top_value / d_keys
 * hold the global answer on every rank.
 *
 * NCCL is bound at run time (dlopen of libnccl.so.2): COGNI_QMM_ERR_NCCL_MISSING without it; a
 * failed NCCL call returns COGNI_QMM_ERR_NCCL_BASE + its ncclResult_t.
 */
int cogni_qmm_sharded_gemv_nccl(void *nccl_comm, int world, int rank, int type, const void *d_w_shard,
                                const float *d_x, float *d_gather, int in_dim, int rows, int batch,
                                int resident, void *stream);
int cogni_qmm_sharded_top1_nccl(void *nccl_comm, int world, int type, const void *d_w_shard,
                                const float *d_x, int in_dim, int rows, int batch, int32_t index_base,
                                void *d_scratch, size_t scratch_bytes, int64_t *d_keys,
                                int32_t *d_top_index, float *d_top_value, void *stream);

/* Lets kernels of the current device store into memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * already-enabled is not an error).  The host needs it once per peer before the first exchange. */
int cogni_qmm_enable_peer_access(int peer_device);

/*
 * Fused lm_head: GEMV over `out_dim` vocabulary rows plus top-1 per batch row, without
 * writing the logits.  Replaces q6_k_gemv_top1_partial_f32 + output_top1_values_reduce_probe
 * (q6k_gemv_probe.ptx:1331; src/ml/cuda/qwen_output_head_runner.cr:530-624, 884-947).
 * Tie rule: highest value, lowest index (src/ml/gguf/qwen35_cpu.cr:2052-2055).
 *   index_base   added to the local row number: a vocab shard passes its first row here
 *   d_scratch    device scratch of at least cogni_qmm_gemv_top1_scratch_bytes() bytes,
 *                8-byte aligned, zero-filled once by the caller before its first use; the
 *                kernel leaves it ready for the next call.  Calls that share one scratch
 *                buffer must be ordered on the device (same stream).
 *   d_top_index  int32 [batch]   global index of the maximum
 *   d_top_value  f32   [batch]   its value
 *   d_top_key    NULL or int64 [batch]: (orderable(value) << 32) | (0xFFFFFFFF - index);
 *                a signed 64-bit MAX over shards' keys yields the global winner under the
 *                same tie rule (used for the cross-GPU reduction).
 */
size_t cogni_qmm_gemv_top1_scratch_bytes(int out_dim, int batch);
int cogni_qmm_gemv_top1(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                        int batch, int32_t index_base, void *d_scratch, size_t scratch_bytes,
                        int32_t *d_top_index, float *d_top_value, int64_t *d_top_key,
                        void *stream);

/*
 * cogni_qmm_gemv_top1 for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its output-head runner allocates its own partial buffers with cuMemAlloc.)
 *
 * A host that gave all of HBM to its own arena at start-up, a plugin whose host only lends it
 * input and output buffers, or a binding that cannot create memory handles at this point has no
 * scratch buffer to pass to cogni_qmm_gemv_top1.  This entry point computes exactly the same
 * result with the scratch kept in a fixed array inside the library; it calls no cudaMalloc,
 * cudaFree or any other allocating routine.  The caller still passes the weights, x and the
 * outputs, with the same meaning and alignment as for cogni_qmm_gemv_top1.
 *
 *   - The array is cogni_qmm_gemv_top1_noalloc_max_scratch() bytes (1 MiB) and every GPU that
 *     loads the library holds it until the process exits, used or not.
 *   - Shapes whose scratch need (cogni_qmm_gemv_top1_scratch_bytes) exceeds that size are
 *     rejected with COGNI_QMM_ERR_LIMIT; a 262144-row vocabulary at batch 16 fits.
 *   - Every call looks up the array's device address for the device that is current (a host
 *     lookup, no device work), so the library survives a host that destroys and re-creates its
 *     context.  Make the first call on a device outside any stream capture.
 *   - A call that is rejected for its arguments does not touch the array.
 *   - All calls on a device share the one array: calls that can overlap on the GPU (different
 *     streams without an ordering between them) race and give wrong answers.  Keep them on one
 *     stream or order them with events.
 */
size_t cogni_qmm_gemv_top1_noalloc_max_scratch(void);
int cogni_qmm_gemv_top1_noalloc(int type, const void *d_w, const float *d_x, int in_dim,
                                int out_dim, int batch, int32_t index_base, int32_t *d_top_index,
                                float *d_top_value, int64_t *d_top_key, void *stream);

/* Decode keys produced by cogni_qmm_gemv_top1 (after a MAX reduction across shards):
 * d_keys int64 [batch] -> d_top_index int32 [batch], d_top_value f32 [batch]. */
int cogni_qmm_top1_unpack_keys(const int64_t *d_keys, int batch, int32_t *d_top_index,
                               float *d_top_value, void *stream);

/*
 * Chunked-prefill GEMM with dequantisation fused into the tile loop:
 *     y[m, n] = sum_k bf16(x[m, k]) * bf16(dequant(W[n, k]))      (fp32 accumulation)
 * The tensor-core replacement for the reference's batched matmul route
 * (Qwen35Metal.matmul with batch > GEMM_BATCH_THRESHOLD, src/ml/gguf/qwen35_metal.cr:75,
 * 10597-10636, 11404-11449; operands rounded to 16-bit, src/ml/gguf/kernels/gemm_q4k.metal:773-776).
 *   d_w      raw GGUF blocks [n_out][k_in], 16-byte aligned
 *   d_x      bf16 [m_rows, k_in] row-major, 16-byte aligned
 *   d_y      [m_rows, n_out] row-major, f32 or bf16 per out_type
 * type: any of the five tensor types.  k_in must be a multiple of 256.
 */
int cogni_qmm_gemm_bf16(int type, const void *d_w, const void *d_x_bf16, void *d_y,
                        int out_type, int m_rows, int n_out, int k_in, void *stream);

/*
 * One-shot host-buffer form with the exact call surface of
 * ML::GGUF::QuantMatmul.matmul_add(x, rows, in_dim, w_raw, w_type, out_dim, bias)
 * (src/ml/gguf/quant_matmul.cr:20-24): uploads, runs the device GEMV, reads back.
 * All pointers are HOST pointers; y receives rows*out_dim floats.  Intended for parity
 * checks and ad-hoc tensors; resident weights use the device entry points above.
 */
int cogni_qmm_matmul_add_host(const float *x, int rows, int in_dim, const void *w_raw,
                              int64_t w_bytes, int type, int out_dim, const float *bias,
                              float *y);

#ifdef __cplusplus
}
#endif
#endif /* COGNI_QMM_H */
