/*
 * b200q — C ABI of the B200 (sm_100a) quantized-GEMM library, libb200q.so.
 *
 * Conventions (the reference project's C++ operator API, op/topk/topk.h:20-28 and
 * op/topk/topk_cuda.cu:229-256, kept as they are):
 *   - free functions, raw DEVICE pointers owned by the caller, explicit integer sizes,
 *     the stream last (NULL = default stream);
 *   - the return value is a cudaError_t as int: 0 on success, cudaErrorInvalidValue (1) for
 *     null pointers, non-positive sizes or unsupported alignment; only argument and launch
 *     errors are reported, the call returns after enqueue and execution errors surface
 *     at the caller's next synchronisation;
 *   - no allocation, no hidden synchronisation; inputs and outputs must not overlap;
 *   - matrices are row-major with K contiguous: A[M,K], B[N,K], C[M,N] = A * B^T
 *     (op/cpu/cpu_ops.h:34-39), fp32 accumulation, output rounded to nearest-even once.
 *
 * The reference snapshot has no foreign-function interface for quantized GEMM; each entry
 * point below names the reference code whose arithmetic it reproduces on the GPU.
 */
#ifndef B200Q_H
#define B200Q_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* FP8 E4M3 GEMM with one fp32 scale per operand:  C(bf16) = (A * B^T) * (scale_a * scale_b).
 * A[M,K], B[N,K] bytes in E4M3 (1.0 = 0x38).  Replaces gemm_mma_cpu (op/cpu/cpu_ops.cpp:95-114)
 * applied to the dequantised operands, with the scale rule of
 * op/test/arch_primitives/ptx_mma_fp8.cu:16-23 (scales multiply the fp32 accumulator).
 * Requires K % 16 == 0 and 16-byte aligned A, B. */
int b200q_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K,
                   float scale_a, float scale_b, void* stream);

/* Grouped (ragged-M) FP8 GEMM: the rows of A[tokens,K] form E consecutive groups of batch_sizes[e] rows, group e is
 * multiplied by its own B[e][N,K]:  C[t,n](bf16) = (A[t,:] . B[e(t)][n,:]) * a_scale[t] * b_scale[e(t)*N + n].
 * The quantized counterpart of the reference's gmm(a, b, batch_sizes, trans_b = True)
 * (op/grouped_gemm/cudaop_grouped_gemm/ops.py:76-83, op/grouped_gemm/csrc/grouped_gemm.cuh:96-328): one persistent
 * launch, the tile -> group map is derived on the device from batch_sizes (DEVICE array of E int64; rows beyond
 * `tokens` are ignored, rows not covered by any group are left untouched in C).  E <= 1024, K % 16 == 0, A and B
 * 16-byte aligned. */
int b200q_gmm_fp8(const void* A, const float* a_scale, const void* B, const float* b_scale, const long long* batch_sizes_dev,
                  void* C, int tokens, int N, int K, int E, void* stream);

/* INT8 GEMM, exact: D[M,N](int32) = A[M,K](s8) * B[N,K](s8)^T + C_in[M,N](int32, or NULL for none), 32-bit wrapping
 * integer arithmetic on the tensor cores (tcgen05 kind::i8).  The S8 case of the reference's integer MMA test as a
 * whole GEMM: signed bytes in two's complement, D = A*B + C with an int32 accumulator
 * (op/test/arch_primitives/ptx_mma_integer.cu:72-92 byte packing, :387-401 reference value).  C_in may equal D.
 * Requires K % 16 == 0 and 16-byte aligned A, B. */
int b200q_gemm_i8(const void* A, const void* B, const void* C_in, void* D, int M, int N, int K, void* stream);

/* Same contraction with per-row and per-column fp32 scales (device arrays):
 * C[m,n] = acc * (row_scale[m] * col_scale[n]); out_f32 != 0 writes fp32 instead of bf16.
 * This is the down projection of the tensor-parallel MLP (row-parallel second GEMM of
 * op/nccl/nccl_mlp_test.cu:170-178) on quantised operands. */
int b200q_gemm_fp8_rowcol(const void* A, const void* B, void* C, int M, int N, int K,
                          const float* row_scale, const float* col_scale, int out_f32, void* stream);

/* Fused gate/up projection + SwiGLU of the MLP: H[M,I](bf16) = silu(g) * u with
 * g = (X * Wgate^T) * row_scale[m] * gate_scale[i], u likewise with Wup / up_scale.
 * X[M,K], Wgate[I,K], Wup[I,K] in E4M3.  Takes the place of the first GEMM + activation
 * kernel of op/nccl/nccl_mlp_test.cu:162-169 (there: SGEMM then gelu_kernel :92-103). */
int b200q_gemm_fp8_swiglu(const void* X, const void* Wgate, const void* Wup, void* H, int M, int I, int K,
                          const float* row_scale, const float* gate_scale, const float* up_scale, void* stream);

/* INT4 weight-only GEMM for decode shapes: Y[M,N](bf16) = X[M,K](bf16) * W^T,
 * w[n,k] = q[n,k] * S[n, k/group].  Wq[N,K/2]: two signed nibbles per byte along K, low
 * nibble = lower K (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S[N,K/group] fp16.
 * Requires group == 128, K % 128 == 0, 16-byte aligned X and Wq. */
int b200q_gemm_w4a16(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K,
                     int group, void* stream);

/* NVFP4 block-scaled GEMM: C(bf16) = ((A.sfa) * (B.sfb)^T) * (global_a * global_b).
 * Aq[M,K/2], Bq[N,K/2]: two E2M1 per byte, low nibble = lower K; SFA[M,K/16], SFB[N,K/16]: one
 * UE4M3 scale per 16 consecutive K, row-major.  Formats, packing and scale rule:
 * op/test/arch_primitives/ptx_mma_fp4.cu:49-65,120-144,285-324.  Requires K % 64 == 0 and 16-byte
 * aligned pointers.  `workspace` is caller-owned scratch of b200q_gemm_nvfp4_workspace_bytes(M,N,K)
 * bytes: the call first rewrites both scale arrays into the blocked layout the tensor core
 * reads (b200q_nvfp4_swizzle_sf), then runs the GEMM on them; all on `stream`. */
int b200q_gemm_nvfp4(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                     int M, int N, int K, float global_a, float global_b, void* workspace, void* stream);
size_t b200q_gemm_nvfp4_workspace_bytes(int M, int N, int K);

/* b200q_gemm_nvfp4 for callers that cannot allocate.  (This entry point has no counterpart in the
 * reference project.)  Some hosts cannot give the call a workspace: a server that handed the whole
 * GPU to its own memory pool at start-up, a latency-critical loop that must stay clear of the
 * allocator's device-wide synchronisation, a plug-in that owns nothing but its operands.  Here the
 * scratch for the rewritten scales is an array inside the library image (8 MiB per GPU that loads
 * the library, kept until exit), so the call performs no allocation of any kind.  Problems whose
 * b200q_gemm_nvfp4_workspace_bytes(M,N,K) exceeds b200q_gemm_nvfp4_static_max_bytes() are refused
 * with cudaErrorInvalidValue and a message on stderr (M = N = K = 8192 just fits).  The first call
 * on a device looks up the array's device address, and, like the first launch of any kernel, makes the
 * driver load the kernels' images and set their attributes, which takes some device memory once: issue
 * one warm-up call per device before any stream capture AND before the host hands the rest of the GPU's
 * memory to its own pool.  From then on a call leaves the amount of free device memory untouched.  All calls
 * on a device share the one array — calls that may overlap on the GPU (several streams) race on
 * it; calls on one stream are safe, and no state has to be cleared between calls. */
int b200q_gemm_nvfp4_static(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                            int M, int N, int K, float global_a, float global_b, void* stream);
size_t b200q_gemm_nvfp4_static_max_bytes(void);

/* The same GEMM on scales that are already in the blocked layout (weights: rewrite once, reuse).
 * Blocked layout: [ceil(rows/128)][K/64] blocks of 512 bytes; inside a block the four scales of
 * row r (K-steps of 16 inside a 64-wide slab) sit at byte (r % 32) * 16 + (r / 32) * 4. */
int b200q_gemm_nvfp4_blocked(const void* Aq, const void* SFA_blocked, const void* Bq, const void* SFB_blocked,
                             void* C, int M, int N, int K, float global_a, float global_b, void* stream);
int b200q_nvfp4_swizzle_sf(const void* sf_rowmajor, void* sf_blocked, int rows, int K, void* stream);
size_t b200q_nvfp4_sf_bytes(int rows, int K);      /* size of one blocked scale array */

/* MXFP8 block-scaled GEMM: C(bf16) = ((A . 2^(sfa-127)) * (B . 2^(sfb-127))^T).  A[M,K], B[N,K]: E4M3 bytes;
 * SFA[M,K/32], SFB[N,K/32]: one UE8M0 scale byte per 32 consecutive K, row-major (value 2^(byte - 127), 0xFF = NaN).
 * This is the reference's kind::mxf8f6f4.block_scale.scale_vec::1X arithmetic
 * (op/test/arch_primitives/ptx_mma_fp8.cu:126-178, scale decoder op/test/arch_primitives/ptx_mma_fp6.cu:344-351) as a
 * whole GEMM.  Requires K % 32 == 0 and 16-byte aligned pointers.  `workspace`: caller-owned scratch of
 * b200q_gemm_mxfp8_workspace_bytes(M,N,K) bytes for the blocked copies of both scale arrays. */
int b200q_gemm_mxfp8(const void* A, const void* SFA, const void* B, const void* SFB, void* C, int M, int N, int K,
                     void* workspace, void* stream);
size_t b200q_gemm_mxfp8_workspace_bytes(int M, int N, int K);
/* The same on scales already in the blocked layout: [ceil(rows/128)][ceil(K/128)] blocks of 512 bytes; inside a
 * block the scales of row r for the four 32-K steps of the 128-K slab sit at bytes (r % 32) * 16 + (r / 32) * 4 + j. */
int b200q_gemm_mxfp8_blocked(const void* A, const void* SFA_blocked, const void* B, const void* SFB_blocked, void* C,
                             int M, int N, int K, void* stream);
int b200q_mxfp8_swizzle_sf(const void* sf_rowmajor, void* sf_blocked, int rows, int K, void* stream);
size_t b200q_mxfp8_sf_bytes(int rows, int K);
int b200q_mxfp8_set_tile_n(int bn);     /* width of the B tile of the MXFP8 GEMM: 256 (default) or 192 */

/* 2:4 structured-sparse FP8 GEMM: C(bf16) = (expand(Acomp, Ameta) * B^T) * (scale_a * scale_b).
 * Acomp[M,K/2] E4M3 keeps the two retained values of every four in order; Ameta[M,K/8]: one
 * nibble per group of four = two ascending 2-bit positions, lower position in bits [1:0],
 * nibbles packed low-first (op/test/arch_primitives/ptx_mma_sparse.cu:53-64,163-184).  The
 * result equals the dense product with the expanded A (ptx_mma_sparse.cu:416-434).
 * Requires K % 128 == 0 and 16-byte aligned pointers. */
int b200q_gemm_sp24_fp8(const void* Acomp, const void* Ameta, const void* B, void* C, int M, int N, int K,
                        float scale_a, float scale_b, void* stream);

/* Tuning knobs.  Every b200q_*_set_* function changes a PROCESS-WIDE setting read by later calls on any
 * device; they are not synchronised with calls in flight on other host threads — set them once at
 * start-up, before the threads that issue work are started.  All of them default to the measured best. */
int b200q_fp8_set_tile_n(int bn);      /* width of the B tile: 0 = chosen per problem (default), 224 or 256 columns */
/* SM partitioning for overlapping the stand-alone all-reduce with GEMMs: the persistent FP8 grids use at
 * most `sms` SMs (0 = all), and the all-reduce kernel asks for `bytes` of shared memory it does not use, so its
 * CTAs cannot share an SM with a GEMM CTA and land on the SMs left free. */
int b200q_fp8_set_sm_limit(int sms);
int b200q_allreduce_set_reserved_smem(int bytes);
int b200q_fp8_set_2cta(int on);        /* FP8 GEMMs on CTA pairs (tcgen05 cta_group::2, 256-row tiles); default on */
int b200q_fp8_set_group(int g);        /* CTA-pair FP8 kernels: tile rows (of 256) that share a pass over the N tiles; 0 = auto */
int b200q_nvfp4_set_group(int g);      /* the same for the CTA-pair NVFP4 kernel */
int b200q_fp8_set_dynamic_tiles(int on);   /* CTA-pair FP8 kernels: tiles handed out by a global counter, so a pair slowed down by a
                                            * co-running kernel takes fewer tiles (default on); off: fixed round-robin shares */
int b200q_fp8_set_tma_store(int on);   /* CTA-pair FP8 kernels: bf16 results via shared memory + TMA stores (default on) */
int b200q_fp8_set_reducer_stride(int stride);   /* fused all-reduce: every stride-th CTA reduces, 1..16 */
int b200q_nvfp4_set_tile_n(int bn);
int b200q_nvfp4_set_2cta(int on);      /* NVFP4 GEMM on CTA pairs (256 x 192 / 256 x 256 tiles per pair) when M > 128 and the
                                        * tile width is not 128; default on */
int b200q_w4a16_set_impl(int impl);     /* 0 = by M (default): streaming CUDA-core GEMV for one token (the older GEMV forms when K is not
                                         * a multiple of 2048 or exceeds 16384), warp-MMA kernel for few tokens, from 64 tokens on (from
                                         * 17 when N >= 8192: the measured crossover) the tcgen05 prefill kernel that keeps the converted weights in tensor memory (group-wise
                                         * partial-sum scaling, product computed transposed);
                                         * 5 / 8 = the streaming GEMV / that prefill kernel wherever they apply;
                                         * 6 / 7 = the prefill kernel that converts through shared memory (the integer offset taken
                                         * out by rows of ones / by the converters);
                                         * 1 = tcgen05 decode kernel; 2 = warp-MMA kernel for every M; 3 / 4 = the two GEMV forms
                                         * (shared memory + dp4a / registers + fp32) for up to 4 tokens */
int b200q_w4a16_set_pdl(int on);        /* programmatic dependent launch of the GEMV / tcgen05 W4A16 kernels (default off):
                                         * the call may start streaming its weights while the previous kernel of the stream
                                         * still runs, so that kernel must not be the one that writes Wq or S */
int b200q_sp24_set_tile_n(int bn);
int b200q_sp24_set_2cta(int on);       /* 2:4-sparse GEMM on CTA pairs (256 x 224 tiles) when M > 128; default on */

/* Activation quantiser: X[rows,cols] bf16 -> Q[rows,cols] E4M3 and S[rows] fp32,
 * S[r] = max(max|X[r,:]| / 448, 2^-126) (1 for a zero row), Q = rn_satfinite(X * (1 / S[r])).  No counterpart in
 * the reference (its MLP is fp32); needed on either side of the FP8 GEMMs.  cols % 8 == 0. */
int b200q_quant_rows_e4m3(const void* X, void* Q, float* S, int rows, int cols, void* stream);

/* Activation quantiser to NVFP4: X[rows,cols] bf16 -> Q[rows,cols/2] (two E2M1 per byte, low nibble = lower K) and
 * one UE4M3 scale per 16 K written directly in the blocked layout of b200q_gemm_nvfp4_blocked
 * (b200q_nvfp4_sf_bytes(rows, cols) bytes; the rows that pad the last 128-row block get zero scales).
 * sf = ue4m3_rn((max|block| / 6) / global_scale), q = e2m1_rn(x * (1 / (decode(sf) * global_scale))).  Formats:
 * op/test/arch_primitives/ptx_mma_fp4.cu:55-65,120-144,293-309; the reference has no quantiser.  cols % 64 == 0,
 * global_scale > 0 (normally max|X| / (6 * 448)); X, SF 16-byte aligned, Q 4-byte aligned. */
int b200q_quant_rows_nvfp4(const void* X, void* Q, void* SF_blocked, int rows, int cols, float global_scale, void* stream);

/* Sum all-reduce of the MLP's fp32 partial outputs over NVLink / NVSwitch, one call per rank, all
 * ranks at the same time: Y(bf16, on every rank) = sum_r P_r, P_r fp32 or (partial_is_bf16) bf16.  Replaces the in-place
 * ncclAllReduce(ncclFloat, ncclSum) of op/nccl/nccl_mlp_test.cu:181-195 with the same contract
 * (fp32 accumulation, bit-identical replicas).  The three pointer arguments are DEVICE arrays of
 * `world` pointers to every rank's partial buffer, output buffer and flag buffer (peer-mapped
 * memory, same layout on every rank; the flag buffer holds b200q_allreduce_signal_bytes() bytes,
 * zeroed once before the first call).  With multicast addresses of the partial and output buffers
 * the switch does the additions and the broadcast; pass NULL for both to use plain peer loads and
 * stores.  `epoch` must grow by one per call, identically on every rank; elems % (8 * world) == 0. */
int b200q_allreduce_to_bf16(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                            void* const* signal_ptrs_dev, const void* partial_multicast, void* out_multicast,
                            int partial_is_bf16, long long elem_offset, long long elems, int rank, int world,
                            unsigned int epoch, unsigned int signal_offset_bytes, int ctas, void* stream);
/* The reduce-scatter half of the same exchange: rank r's call sums elements [elem_offset + r * elems / world,
 * elem_offset + (r + 1) * elems / world) of every rank's partial buffer (same arithmetic and rounding) and stores
 * them to the same range of its OWN output buffer only; nothing is broadcast and there is no end barrier.  A
 * caller completes the other ranges with device-to-device copies from the peers' output buffers (copy engines:
 * no SM is taken from a GEMM running beside them), ordered behind a b200q_rank_barrier on the same stream.
 * Together they are the ncclAllReduce of op/nccl/nccl_mlp_test.cu:181-195 split into its two phases. */
int b200q_reduce_scatter_to_bf16(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                 void* const* signal_ptrs_dev, const void* partial_multicast, int partial_is_bf16,
                                 long long elem_offset, long long elems, int rank, int world, unsigned int epoch,
                                 unsigned int signal_offset_bytes, int ctas, void* stream);
/* out[e] = bf16( sum_i src_i[e] ) for `n` arrays of this device (fp32 or bf16), fp32 accumulation in index order,
 * one round-to-nearest-even: the arithmetic of the exchange alone, for callers that move the ranks' partial sums
 * with copy engines (device-to-device copies behind b200q_rank_barrier) so that no SM is busy with NVLink traffic
 * beside a running GEMM.  `srcs_dev`: device array of n pointers, 16-byte aligned; elems % 8 == 0. */
int b200q_sum_to_bf16(const void* const* srcs_dev, int n, int src_is_bf16, void* out, long long elems, int ctas, void* stream);
int b200q_allreduce_set_unroll(int unroll);     /* tuning knob: independent reductions in flight per thread, 1..8 */
int b200q_allreduce_set_threads(int threads);   /* tuning knob: threads per CTA of the all-reduce kernel, 128/256/512 */
size_t b200q_allreduce_signal_bytes(void);

/* A barrier over the ranks, in stream order: the kernel ends on this rank once every rank's call with the same
 * `epoch` (growing by one per call) has started, i.e. once everything enqueued before it on every rank's
 * launching stream has completed.  `signal_ptrs_dev`: device array of `world` pointers to every rank's flag words
 * (peer-mapped, b200q_rank_barrier_signal_bytes() bytes from signal_offset_bytes on, zeroed once).  Bounded like
 * every wait of the library (cross-rank limit; status site 16).  Used to order copies between ranks' buffers;
 * it plays the part of the stream synchronisation around ncclAllReduce in op/nccl/nccl_mlp_test.cu:181-195. */
int b200q_rank_barrier(void* const* signal_ptrs_dev, int rank, int world, unsigned int epoch,
                       unsigned int signal_offset_bytes, void* stream);
size_t b200q_rank_barrier_signal_bytes(void);

/* The MLP's row-parallel down projection with the all-reduce fused into the same kernel (one
 * kernel in place of GEMM -> ncclAllReduce, op/nccl/nccl_mlp_test.cu:170-195): every rank calls it
 * at the same time; the kernel writes partial tiles (fp32, or bf16 with partial_is_bf16) to `partial_local` (this rank's entry of
 * partial_ptrs_dev), and while later row groups are still being multiplied its reducer warps sum
 * finished groups across ranks through NVSwitch and broadcast the bf16 result to every rank's
 * output.  Pointer-array, multicast, epoch and flag arguments as for b200q_allreduce_to_bf16;
 * the flag buffer needs b200q_fused_allreduce_flag_bytes() bytes from flag_offset_bytes on (zeroed
 * once), `counters_local` is b200q_fused_allreduce_counter_bytes() of this rank's own memory. */
int b200q_gemm_fp8_rowcol_allreduce(const void* A, const void* B, void* partial_local, int M, int N, int K,
                                    const float* row_scale, const float* col_scale,
                                    const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                    void* const* flag_ptrs_dev, const void* partial_multicast, void* out_multicast,
                                    int partial_is_bf16, void* counters_local, unsigned int flag_offset_bytes,
                                    unsigned int epoch, int rank, int world, void* stream);
size_t b200q_fused_allreduce_flag_bytes(void);
size_t b200q_fused_allreduce_counter_bytes(void);

/* All ranks of a small world inside ONE cooperative launch on ONE device, for exercising the flag protocol
 * and the reducers where only one GPU is at hand (tests): CTAs [r * ctas_per_rank, (r + 1) * ctas_per_rank)
 * act as rank r.  The pointer tables are device arrays as above, every buffer in this device's memory; plain
 * loads/stores only (no multicast).  Fails with cudaErrorCooperativeLaunchTooLarge instead of waiting when
 * the CTAs of all ranks cannot be resident together.  Same arithmetic as the per-rank entry points
 * (op/nccl/nccl_mlp_test.cu:181-195: fp32 sum in rank order, replicas identical). */
int b200q_allreduce_to_bf16_one_device(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                       void* const* signal_ptrs_dev, int partial_is_bf16, long long elem_offset,
                                       long long elems, int world, unsigned int epoch, unsigned int signal_offset_bytes,
                                       int ctas_per_rank, void* stream);
/* The reduce-scatter half in the same one-launch form: "rank" r's CTAs write elements
 * [elem_offset + r * elems / world, elem_offset + (r + 1) * elems / world) of the sum to out_ptrs_dev[r] only. */
int b200q_reduce_scatter_to_bf16_one_device(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                            void* const* signal_ptrs_dev, int partial_is_bf16, long long elem_offset,
                                            long long elems, int world, unsigned int epoch,
                                            unsigned int signal_offset_bytes, int ctas_per_rank, void* stream);
/* The same for b200q_gemm_fp8_rowcol_allreduce (world <= 4).  A_host / B_host / row_scale_host / partial_host /
 * counters_host are HOST arrays of `world` device pointers (rank r's operands, its partial buffer = entry r of
 * partial_ptrs_dev, its counter block); col_scale is shared; the three *_dev tables are device arrays. */
int b200q_gemm_fp8_rowcol_allreduce_one_device(const void* const* A_host, const void* const* B_host,
                                               const float* const* row_scale_host, const float* col_scale,
                                               void* const* partial_host, void* const* counters_host,
                                               const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                               void* const* flag_ptrs_dev, int M, int N, int K, int partial_is_bf16,
                                               unsigned int flag_offset_bytes, unsigned int epoch, int world,
                                               int ctas_per_rank, void* stream);

/* Reads (and optionally clears) the device status word of the current device into *host_out.
 * 0 = no kernel of this library gave up on a bounded wait.  Otherwise bit 31 is set, bits [30:24] name the
 * wait that ran out (1-7, 21-28: an mbarrier inside a GEMM; 5, 6: a flag of the fused all-reduce; 16, 17:
 * the start / end barrier of the stand-alone all-reduce) and bits [23:0] the CTA.  A kernel that gave up
 * returns early: ITS OUTPUT IS UNDEFINED (stale or partly written) and must not be used.  Synchronises the
 * device. */
int b200q_status(unsigned int* host_out, int clear);
/* Limit of the bounded waits on the current device, in milliseconds (1 .. 600000).  kind 0: waits on
 * something inside the GPU (mbarriers; default 2000); kind 1: waits on a flag that another rank raises
 * (the all-reduce barriers and the fused reducers; default 10000 — ranks may legitimately be seconds apart
 * on a first call or after a host stall, and a rank that gives up leaves an undefined result).  Synchronous. */
int b200q_set_wait_limit_ms(int kind, int ms);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
