/*
 * kernelcore_b200.h -- C ABI of the B200 implementation of Kernelcore's quantized-LLM hot path.
 *
 * Plain pointers and sizes only.  Every pointer named "device" is CUDA device memory of the current
 * device; `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Every
 * function returns an int status whose values are the reference's kc::Error codes
 * (include/kernelcore/error.hpp:8-25 of the reference): 0 = Success, 2 = InvalidValue,
 * 5 = InvalidPointer, 7 = UnsupportedOperation, 11 = LaunchFailure, ...  Op entry points only enqueue
 * work; they never synchronise and never allocate.
 *
 * Each declaration cites the reference interface it stands in for (path inside the reference project).
 */
#ifndef KERNELCORE_B200_H
#define KERNELCORE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library ------------------------------------------------------------------------------- */
/* ABI revision and build arch string ("sm_100a"). */
int         kcb_abi_version(void);
const char* kcb_build_arch(void);
/* Text for a status code: kcGetErrorString, include/kernelcore/api.hpp:80. */
const char* kcb_error_string(int status);

/* ---- runtime: the C layer under the reference's kc* functions (include/kernelcore/api.hpp:15-85) -----
 * Each kcb_x below is what kcX forwards to; handles are opaque pointers; `kind` is kc::CopyKind
 * (0 H2D, 1 D2H, 2 D2D, 3 H2H).  A NULL stream handle means the current device's default stream, on
 * which launches are synchronous (api.hpp:34-35). */
int kcb_init(void);                                   /* kcInit, api.hpp:16 */
int kcb_shutdown(void);                               /* kcShutdown, api.hpp:17 */
int kcb_device_reset(void);                           /* kcDeviceReset, api.hpp:18 */
int kcb_get_device_count(int* count);                 /* kcGetDeviceCount, api.hpp:21 */
int kcb_get_device_properties(char* name128, unsigned* sm_count, size_t* total_memory, int device); /* api.hpp:22 */
int kcb_set_device(int device);                       /* kcSetDevice, api.hpp:23 (per calling thread) */
int kcb_get_device(int* device);                      /* kcGetDevice, api.hpp:24 */
int kcb_device_synchronize(void);                     /* kcDeviceSynchronize, api.hpp:25 */
int kcb_malloc(void** ptr, size_t bytes);             /* kcMalloc, api.hpp:28 */
int kcb_free(void* ptr);                              /* kcFree, api.hpp:29 */
int kcb_memcpy(void* dst, const void* src, size_t bytes, int kind); /* kcMemcpy, api.hpp:30 */
int kcb_memset(void* dst, int value, size_t bytes);   /* kcMemset, api.hpp:31 */
/* LaunchContext::checkDeviceRange (include/kernelcore/kernel_registry.hpp:27-33): 0 iff the range lies
 * inside one live allocation of the current device. */
int kcb_check_range(const void* ptr, size_t bytes);
int kcb_register_kernel(const void* kernel_entry);    /* kcRegisterKernel, api.hpp:33 (kc::KernelEntry*) */
/* kcLaunchKernel / kcLaunchKernelChunked, api.hpp:35-39: typed_args points at the kernel's llm::*Args
 * struct (llm/llm_kernels.hpp), host memory. */
int kcb_launch_kernel(const char* name, const void* typed_args, void* stream);
/* The built-in kernel table (every name of llm::registerKernels, llm/llm_kernels.cpp:1016-1062, plus vector_add and
 * flash_attn_f16): number of entries and the name of entry i (NULL outside the range).  No device needed. */
int kcb_kernel_count(void);
const char* kcb_kernel_name(int i);
int kcb_stream_create(void** stream);                 /* kcStreamCreate, api.hpp:42 */
int kcb_stream_destroy(void* stream);                 /* kcStreamDestroy, api.hpp:43 */
int kcb_stream_synchronize(void* stream);             /* kcStreamSynchronize, api.hpp:44 */
int kcb_stream_query(void* stream);                   /* kcStreamQuery, api.hpp:45 */
int kcb_launch_host_func(void* stream, void (*fn)(void*), void* user); /* kcLaunchHostFunc, api.hpp:46 */
int kcb_event_create(void** event);                   /* kcEventCreate, api.hpp:47 */
int kcb_event_destroy(void* event);                   /* kcEventDestroy, api.hpp:48 */
int kcb_event_record(void* event, void* stream);      /* kcEventRecord, api.hpp:49 */
int kcb_event_synchronize(void* event);               /* kcEventSynchronize, api.hpp:50 */
int kcb_event_query(void* event);                     /* kcEventQuery, api.hpp:51 */
int kcb_event_elapsed_ms(void* start, void* stop, float* ms); /* device time between two recorded events;
                                                         the reference times with host clocks (app/llm_bench.cpp:207-262) */
int kcb_stream_wait_event(void* stream, void* event); /* kcStreamWaitEvent, api.hpp:52 */
int kcb_stream_begin_capture(void* stream);           /* kcStreamBeginCapture, api.hpp:59 */
int kcb_stream_end_capture(void* stream, void** graph); /* kcStreamEndCapture, api.hpp:60 */
int kcb_graph_launch(void* graph, void* stream);      /* kcGraphLaunch, api.hpp:65 */
int kcb_graph_destroy(void* graph);                   /* kcGraphDestroy, api.hpp:70 */
int kcb_stream_concurrent(void* stream, int begin);   /* kcStreamConcurrentBegin/End, api.hpp:68-69 */
int kcb_get_last_fault(void* fault_info);             /* kcGetLastFault, api.hpp:79 (kc::FaultInfo*) */
/* Test hook: the next runtime call on the current device that waits for or enqueues device work, and itself
 * succeeds, reports this CUDA error code instead (once).  Lets a test drive KernelFault -> ContextPoisoned ->
 * kcDeviceReset (src/runtime.cpp:238-252, 602-615 of the reference) without making a kernel fail. */
int kcb_test_inject_device_error(int cuda_error);
const char* kcb_last_error_detail(void);              /* kcGetLastErrorDetail, api.hpp:85 */
/* The cudaStream_t behind a stream handle, for callers that mix kcb_* op entry points with runtime streams. */
void* kcb_stream_native(void* stream);

/* Number of bounded device-side waits (mbarrier polls of the bulk-copy pipelines) that gave up since
 * the library was loaded; 0 in a healthy process.  Synchronous.  No counterpart in the reference: its
 * fault reporting is kcGetLastFault (include/kernelcore/api.hpp:79). */
unsigned kcb_tma_timeouts(void);

/* ---- weight layouts -------------------------------------------------------------------------
 * Q4_K matrices live on the device as canonical GGUF super-blocks, row-major: rows*(k/256) blocks
 * of 144 bytes.  Q6_K matrices live as four planes (ql | qh | scales | d) of the same total size,
 * rows*(k/256)*210 bytes; kcb_q6k_to_planes / kcb_q6k_from_planes convert from / to canonical GGUF
 * blocks on the device.  These replace the host-side 8-row interleaving of
 * llm::ref::repackQ4K / repackQ6K (llm/llm_reference.cpp:385-411) that the reference's loaders run
 * (llm/gguf_model.cpp:29-49, integrations/llama.cpp/.../ggml-kernelcore.cpp:175-190); the inverse
 * serves get_tensor (ggml-kernelcore.cpp:192-206). */
size_t kcb_kquant_bytes(int rows, int k, int q6);
int    kcb_q6k_to_planes(const void* gguf_blocks_dev, void* planes_dev, int rows, int k, void* stream);
int    kcb_q6k_from_planes(const void* planes_dev, void* gguf_blocks_dev, int rows, int k, void* stream);

/* Bit-exact dequantisation to fp32 [rows][k]: llm::ref::dequantRowQ4K / dequantRowQ6K
 * (llm/llm_reference.cpp:342-383), used for embedding rows (llm/gguf_model.cpp:96-104). */
int kcb_dequant_q4k(const void* w_dev, float* out_dev, int rows, int k, void* stream);
int kcb_dequant_q6k(const void* planes_dev, float* out_dev, int rows, int k, void* stream);

/* ---- activation quantizers ------------------------------------------------------------------- */
/* kernel "quantize_q8x4", llm::QuantizeArgs (llm/llm_kernels.hpp:51-57; kernels/llm/quantize_q8x4.cu:8-41):
 * count blocks of 32 floats -> xq[count*8] packed int8 words, xd[count*2] = {scale, sum of q}. */
int kcb_quantize_q8x4(const float* x_dev, int32_t* xq_dev, float* xd_dev, int count, void* stream);
/* kernels "quantize_cols" / "quantize_cols_k", llm::QuantizeColsArgs (llm/llm_kernels.hpp:273-283):
 * ncols columns of k floats -> slots of 11*k/32 ints (per-32 scales) or 85*k/256 ints (per-256). */
int kcb_quantize_cols(const float* x_dev, int32_t* q_dev, int k, int ncols, void* stream);
int kcb_quantize_cols_k(const float* x_dev, int32_t* q_dev, int k, int ncols, void* stream);

/* ---- decode matvec ---------------------------------------------------------------------------- */
/* kernels "matvec_q4k_q8" / "matvec_q6k_q8", llm::MatvecQ4Q8Args (llm/llm_kernels.hpp:59-70;
 * kernels/llm/matvec_q4k_q8.cu:33-88, matvec_q6k_q8.cu:33-105): y[rows] = W x with x given as the
 * Q8 blocks quantize_q8x4 wrote.  k % 256 == 0, k <= 32768. */
int kcb_matvec_q4k_q8(const void* w_dev, const int32_t* xq_dev, const float* xd_dev, float* y_dev, int rows, int k,
                      void* stream);
int kcb_matvec_q6k_q8(const void* planes_dev, const int32_t* xq_dev, const float* xd_dev, float* y_dev, int rows,
                      int k, void* stream);
/* Both of the above on the same activations in one launch: y4 = W4 x (Q4_K), y6 = W6 x (Q6_K planes) -- the q|k and
 * v projections of a Q4_K_M layer (the three Backend::matvec calls of llm::decodeToken on the attention input), the Q6_K
 * output bit-identical to its own launch, the Q4_K output to 1e-6 (same integer dot products, fp32 sums in another order).  k <= 4096 and at most 6144 rows each; beyond that KCB_UNSUPPORTED_OPERATION (7),
 * and the caller launches them separately (larger matrices stream better through the bulk-copy kernel). */
int kcb_matvec_q4k_q6k_pair_q8(const void* w4_dev, float* y4_dev, int rows4, const void* planes6_dev, float* y6_dev, int rows6,
                               const int32_t* xq_dev, const float* xd_dev, int k, void* stream);
/* The same product on fp32 activations: y = dequant(W) x with fp32 accumulation, the quantity the
 * reference's tests call "dequantized floats" (tests/test_llm_kernels.cpp:228-236).  k <= 12288. */
int kcb_matvec_q4k_f32(const void* w_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream);
int kcb_matvec_q6k_f32(const void* planes_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream);

/* ---- prompt matmul -------------------------------------------------------------------------------- */
/* kernels "matmul_q4k_q8x4/x8", "matmul_q6k_q8x4/x8" (q8k = 0: per-32 slots of 11*k/32 ints per column) and
 * "matmul_q4k_q8kx4/x8", "matmul_q6k_q8kx4/x8" (q8k = 1: per-256 slots of 85*k/256 ints), llm::MatmulKQ8Args
 * (llm/llm_kernels.hpp:255-271): Y[c*rows + r] for ncols activation columns.  Per-256 slots with rows % 128 == 0,
 * k % 1024 == 0 and at least 16 columns run on the tensor cores (tcgen05, int8) in one pass, every output
 * bit-identical to llm::ref::matvecQ4KQ8K / matvecQ6KQ8K (llm/llm_reference.cpp:529-596); other cases on CUDA cores. */
int kcb_matmul_kq_q8(const void* w_dev, const int32_t* slots_dev, float* y_dev, int rows, int k, int ncols, int q6, int q8k,
                     void* stream);
/* The same with a caller-owned device workspace of kcb_matmul_tc_workspace_bytes(rows, k, ncols) bytes: where few
 * tiles would leave SMs idle, the tensor-core launch then contracts K in kcb_matmul_tc_k_slices slices that a second
 * kernel adds in slice order (outputs within ~1e-6 of the one-pass result, deterministic).  A null or smaller
 * workspace means one pass.  Nothing is allocated by either call, inside or outside stream capture. */
int kcb_matmul_kq_q8_ws(const void* w_dev, const int32_t* slots_dev, float* y_dev, int rows, int k, int ncols, int q6, int q8k,
                        void* workspace_dev, size_t workspace_bytes, void* stream);
size_t kcb_matmul_tc_workspace_bytes(int rows, int k, int ncols);
/* The reference's synthetic weight formats and fp16 matmul (kernels/llm/matvec_q8.cu, matvec_q4.cu, matvec_q4x8.cu,
 * matvec_q4x8_q8.cu / _q8x2.cu, matmul_f16.cu; layouts llm/llm_kernels.hpp:24-70, :284-296).  Bit-identical to
 * llm::ref::matvecQ8 / matvecQ4 / matvecQ4x8 / matvecQ4x8Q8 / matmulF16.  `interleaved` selects the 8-row
 * interleaved layout of llm::ref::repackQ4x8 (rows % 8 == 0); qw of kcb_matvec_q4x8_q8 is llm::ref::repackQ4x8Q8's
 * stream, of kcb_matmul_f16 llm::ref::repackF16's. */
int kcb_matvec_q8w(const int8_t* q_dev, const float* scales_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream);
int kcb_matvec_q4w(const uint8_t* qs_dev, const float* scales_dev, const float* x_dev, float* y_dev, int rows, int k, int interleaved,
                   void* stream);
int kcb_matvec_q4x8_q8(const int32_t* qw_dev, const int32_t* xq_dev, const float* xd_dev, float* y_dev, int rows, int k, void* stream);
int kcb_matmul_f16(const int32_t* qw_dev, const float* x_dev, float* y_dev, int rows, int k, int ncols, void* stream);
/* Bounded waits of the tensor-core kernel that expired since load (0 in a healthy process); synchronous. */
unsigned kcb_tc_timeouts(void);
/* How many K slices kcb_matmul_kq_q8_ws contracts a tensor-core shape in when given its workspace: 1 = one pass,
 * more = slices added in order by a second kernel.  0 for shapes that path does not take (rows % 128, k % 1024).
 * Pure host arithmetic. */
int kcb_matmul_tc_k_slices(int rows, int k, int ncols);

/* ---- row-sharded matvec across GPUs (no counterpart in the reference, which is single-device) -------------
 * One process per GPU, rank r owning `rows` consecutive rows of a Q6_K matrix (its own planes).  The kernel
 * writes each result to y_local[row] and, through NVLink peer mappings, to y_peers[i][row] for the npeers <= 7
 * other ranks: y_local / y_peers[i] point at THIS rank's first row inside each rank's full-length output, so
 * the all-gather of the logits rides on the matvec's stores.  rows % 8 == 0, k <= 4096. */
int kcb_matvec_q6k_q8_gather(const void* planes_dev, const int32_t* xq_dev, const float* xd_dev, float* y_local,
                             float* const* y_peers, int npeers, int rows, int k, void* stream);
/* Cross-GPU step barrier for the gathered output: flags[i] is rank i's array of `world` 32-bit counters (peer
 * mapped, zero-initialised).  Rank `rank` stores `epoch` (release, system scope) into flags[i][rank] for all i
 * and waits until flags[rank][i] >= epoch for all i.  The wait is bounded; an expiry is counted in
 * kcb_peer_timeouts() and the kernel returns.  Use a fresh, increasing epoch per step. */
int kcb_peer_barrier(unsigned* const* flags, int rank, int world, unsigned epoch, void* stream);
unsigned kcb_peer_timeouts(void);
/* Failure handling of the cross-GPU waits (kcb_peer_barrier and the barrier inside kcb_matvec_q6k_f32x_sharded).  A
 * wait polls at most `polls` times (0 restores the default, about a second) and then gives up: the expiry is counted,
 * the kernel returns, and the group is marked broken so that later barriers announce themselves, poll once and return
 * -- a rank whose peer is gone does not wait out every step.  The context stays usable.  kcb_peer_reset clears the
 * count and the mark once the host has dealt with the failure.  Both calls are synchronous.  (The reference detects a
 * lost worker on the host, src/runtime.cpp:238-252; this is the device-side half a multi-GPU step needs.) */
int kcb_peer_set_poll_limit(unsigned polls);
int kcb_peer_reset(void);
/* The whole sharded step in ONE kernel launch: x (fp32, k floats) is quantized to Q8 blocks of 32 inside the
 * kernel (quantize_q8x4's arithmetic), the row shard is multiplied, results go to y_local and to the npeers other
 * ranks' outputs, and -- world > 1 -- the last CTA to finish runs the step barrier on `flags` (as
 * kcb_peer_barrier).  counters: two zero-initialised device words owned by this rank (epoch, finished CTAs); NULL
 * when world == 1.  ev_before / ev_after: optional cudaEvent_t recorded around the launch on `stream`.  With
 * npeers == 0 and world == 1 this is Backend::matvec for one Q6_K matrix (llm/llm_model.cpp:385-397) in a single
 * launch.  rows % 8 == 0, k <= 4096, x_dev 16-byte aligned. */
int kcb_matvec_q6k_f32x_sharded(const void* planes_dev, const float* x_dev, float* y_local, float* const* y_peers, int npeers,
                                unsigned* const* flags, unsigned* counters, int rank, int world, int rows, int k, void* ev_before,
                                void* ev_after, void* stream);

/* No counterpart in the reference.  y = W x for a Q4_K matrix and fp32 x like kcb_quantize_q8x4 followed by
 * kcb_matvec_q4k_q8, but the 8-bit activation scratch lives in a fixed device array inside the library, so
 * the call allocates nothing and needs no caller scratch -- for hosts that may not allocate device memory
 * at call time (plugins under an application that owns all buffers, allocation-free serving loops).
 * k % 256 == 0 and k <= kcb_static_scratch_max_k() (16384), else InvalidValue.  The first call on a device
 * looks up the array's address and loads the kernels (the CUDA runtime may allocate for that): make one warm-up
 * call before any stream capture and before memory is counted; later calls only launch.  All calls share the
 * one array per GPU: calls whose GPU work may overlap race; keep them on one stream. */
int kcb_matvec_q4k_f32x_static(const void* w_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream);
int kcb_static_scratch_max_k(void);

/* ---- normalisation ------------------------------------------------------------------------------- */
/* kernel "rms_norm", llm::RmsNormArgs (llm/llm_kernels.hpp:118-125; kernels/llm/rms_norm.cu:2-11):
 * y[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w for `rows` rows of n. */
int kcb_rms_norm(const float* x_dev, const float* w_dev, float* y_dev, int n, int rows, float eps, void* stream);
/* kernel "add_rms_norm", llm::AddRmsNormArgs (llm/llm_kernels.hpp:72-80): x += t; y = norm(x) * w, one row. */
int kcb_add_rms_norm(float* x_dev, const float* t_dev, const float* w_dev, float* y_dev, int n, float eps, void* stream);
/* kernels "add_sumsq" / "norm_q8x4", llm::AddSumsqArgs / NormQ8Args (llm/llm_kernels.hpp:91-106):
 * x += t with per-32 partial sums of squares into the scratch q (11*nb ints); then
 * norm(x) * w quantized into q.  kcb_add_norm_q8x4 runs both in one launch (Backend::addRmsNormQuant,
 * llm/llm_model.cpp:417-423). */
int kcb_add_sumsq(float* x_dev, const float* t_dev, int32_t* q_dev, int nb, void* stream);
int kcb_norm_q8x4(const float* x_dev, const float* w_dev, int32_t* q_dev, int nb, float eps, void* stream);
int kcb_add_norm_q8x4(float* x_dev, const float* t_dev, const float* w_dev, int32_t* q_dev, int nb, float eps, void* stream);
/* ggml-graph forms, rows of n (n % 256 == 0), one scratch slot of 11*n/32 ints per row:
 * kernels "add_sumsq_f" (AddSumsqFArgs), "sumsq_part" (SumsqPartArgs), "norm_mul_q8_f" (NormMulQ8Args)
 * and "norm_mul_q8k_f" (per-256 slots of 85*n/256 ints in q, partial sums in sq)
 * (llm/llm_kernels.hpp:170-216). */
int kcb_add_sumsq_f(const float* a_dev, const float* b_dev, float* out_dev, int32_t* q_dev, int n, int rows, void* stream);
int kcb_sumsq_part(const float* x_dev, int32_t* q_dev, int n, int rows, void* stream);
int kcb_norm_mul_q8_f(const float* x_dev, const float* w_dev, float* y_dev, int32_t* q_dev, int n, int rows, float eps, void* stream);
int kcb_norm_mul_q8k_f(const float* x_dev, const float* w_dev, float* y_dev, int32_t* q_dev, const int32_t* sq_dev, int n,
                       int rows, float eps, void* stream);

/* ---- SwiGLU and elementwise ------------------------------------------------------------------------ */
/* kernel "silu_mul", llm::SiluMulArgs (llm/llm_kernels.hpp:248-253). */
int kcb_silu_mul(const float* g_dev, const float* u_dev, float* out_dev, int count, void* stream);
/* kernel "silu_mul_q8x4", llm::SiluMulQ8Args (llm/llm_kernels.hpp:108-116): count blocks of 32. */
int kcb_silu_mul_q8x4(const float* g_dev, const float* u_dev, int32_t* xq_dev, float* xd_dev, int count, void* stream);
/* kernels "silu_mul_q8x4f" / "silu_mul_q8kf", llm::SiluMulQ8FArgs (llm/llm_kernels.hpp:200-216): cols columns
 * of n, fp32 y stored, slots per column. */
int kcb_silu_mul_q8x4f(const float* g_dev, const float* u_dev, float* y_dev, int32_t* q_dev, int n, int cols, void* stream);
int kcb_silu_mul_q8kf(const float* g_dev, const float* u_dev, float* y_dev, int32_t* q_dev, int n, int cols, void* stream);
/* kernel "mul_rows", llm::MulRowsArgs (llm/llm_kernels.hpp:146-153); kernel "vector_add",
 * kc::kernels::VectorAddArgs (include/kernelcore/kernels.hpp:10-16). */
int kcb_mul_rows(const float* x_dev, const float* w_dev, float* y_dev, int n, int count, void* stream);
int kcb_vector_add(const float* a_dev, const float* b_dev, float* out_dev, int count, void* stream);

/* ---- RoPE ----------------------------------------------------------------------------------------- */
/* kernels "rope" / "rope_ff", llm::RopeArgs / RopeFFArgs (llm/llm_kernels.hpp:127-144): in place, adjacent
 * pairs, one position; ff_dev may be NULL (no frequency factors). */
int kcb_rope(float* x_dev, const float* ff_dev, int pairs_per_head, int pos, int count, float log2_base, void* stream);
/* kernel "rope_ggml", llm::RopeGgmlArgs (llm/llm_kernels.hpp:155-168): out of place, per-token positions,
 * NORM or NEOX pairing; ff_dev may be NULL. */
int kcb_rope_ggml(const float* x_dev, float* y_dev, const int32_t* pos_dev, const float* ff_dev, int head_dim, int n_head,
                  int n_tokens, float log2_base, int neox, void* stream);

/* ---- attention over the decode loop's fp32 cache -------------------------------------------------------
 * llm::AttnDims as seven ints {n_heads, ctx, head_dim, kv_stride, group, ctx_pad, k_stride}
 * (llm/llm_kernels.hpp:14-23), passed by value instead of a device int[7]. */
/* kernel "kv_append", llm::KvAppendArgs (llm/llm_kernels.hpp:234-241): writes position ctx-1. */
int kcb_kv_append(const float* k_dev, const float* v_dev, float* kt_dev, float* vc_dev, const int* attn_dims7, void* stream);
/* kernels "attn_scores", "softmax", "attn_values" (llm/llm_kernels.hpp:218-247). */
int kcb_attn_scores(const float* q_dev, const float* kt_dev, float* scores_dev, const int* attn_dims7, float scale, void* stream);
int kcb_softmax(float* x_dev, int n, int stride, int rows, void* stream);
int kcb_attn_values(const float* p_dev, const float* v_dev, float* out_dev, const int* attn_dims7, void* stream);

/* ---- fp16 KV cache (the ggml backend's path) ----------------------------------------------------------- */
/* kernel "set_rows_f16", llm::SetRowsF16Args (llm/llm_kernels.hpp:298-311). */
int kcb_set_rows_f16(const float* src_dev, const int64_t* idx_dev, void* dst_dev, int pairs, int rows, int src_row,
                     int dst_row, int dst_rows, void* stream);
/* kernels "fa_scores" + "fa_max" + "fa_exp" + "fa_values" as one launch; fa_dims15 = llm::FaDims in
 * faDimsInts order (llm/llm_kernels.hpp:316-338), host memory.  mask_dev may be NULL when has_mask == 0. */
int kcb_flash_attn_f16(const float* q_dev, const void* k_dev, const void* v_dev, const void* mask_dev, float* out_dev,
                       const int* fa_dims15, float scale, void* stream);

/* ---- decoder model and decode loop ----------------------------------------------------------------------
 * C view of llm::Model / llm::decodeToken / llm::makeKcBackend (llm/llm_model.hpp:100-207 of the reference;
 * model assembly as llm/gguf_model.cpp:51-106).  Weights are given as canonical GGUF blocks in HOST
 * memory (fmt 4 = Q4_K, 6 = Q6_K); the library packs and uploads them to the current device.  Embeddings
 * are tied to lm_head.  q_norm / k_norm are read only when qk_norm != 0. */
typedef struct { const void* blocks; int rows, k, fmt; } kcb_mat;
typedef struct {
    kcb_mat wq, wk, wv, wo, wg, wu, wd;
    const float* attn_norm; const float* ffn_norm; const float* q_norm; const float* k_norm;
} kcb_layer;
typedef struct {
    int hidden, inter, n_layers, heads, kv_heads, head_dim, vocab, max_ctx;
    float eps, rope_base;
    int neox, qk_norm;
    const kcb_layer* layers; const float* out_norm; kcb_mat lm_head; const float* rope_ff;
} kcb_model_desc;
/* Needs kcb_init.  The host blocks of lm_head must stay valid for the model's lifetime (embedding lookups
 * read them).  graphs != 0: each token's launches are recorded and run as one CUDA graph. */
int kcb_model_create(const kcb_model_desc* desc, int graphs, void** model);
/* llm::decodeToken: one decode step for `token` at position pos (0-based, == tokens decoded so far).
 * logits_host (vocab floats) may be NULL; argmax may be NULL.  token < 0 only for synthetic models (below). */
int kcb_model_decode(void* model, int token, int pos, float* logits_host, int* argmax);
int kcb_model_destroy(void* model);
/* llm::buildModels + llm::allocActs (llm/llm_model.cpp:217-283 of the reference): a random-weight model of the shape in
 * desc (its pointer members are not read) in a synthetic format -- weights 0 = Q8, 1 = Q4, 2 = Q4X8, 3 = Q4X8Q8 --
 * whose values are, for equal seeds, the reference's bit for bit; the KV caches start filled, so a step at any position
 * is defined.  Such a model has no embedding table: kcb_model_decode takes token < 0 and starts from the vector drawn
 * from start_seed. */
int kcb_model_create_synthetic(const kcb_model_desc* desc, int weights, unsigned long long model_seed,
                               unsigned long long start_seed, int graphs, void** model);
/* Text of the last exception a kcb_model_* call on this thread turned into a status code (the reference's
 * decode loop reports failures as C++ exceptions, llm/llm_model.cpp:91-97). */
const char* kcb_model_last_error(void);

/* ---- host-buffer matvec pipe ------------------------------------------------------------------------------
 * For callers whose activations and results stay in host memory, as everything does in the reference
 * (Backend::matvec, llm/llm_model.cpp:385-397, reads x and writes y in process memory).  submit() enqueues
 * x_host -> device, the single-launch Q6_K matvec and y -> y_host on two internal streams and returns at once; the
 * read-back of one call overlaps the kernel of the next (two slots).  y_host of a call is complete after
 * kcb_host_matvec_sync, or once the second following submit has returned.  Pin the host buffers.  rows % 8 == 0,
 * k <= 4096; planes_dev may differ from call to call (same shape). */
int kcb_host_matvec_create(int rows, int k, void** pipe);
int kcb_host_matvec_submit(void* pipe, const void* planes_dev, const float* x_host, float* y_host);
int kcb_host_matvec_sync(void* pipe);
int kcb_host_matvec_destroy(void* pipe);

/* ---- GGUF files (llm/gguf.cpp:79-139 reader, llm/gguf_model.cpp:51-106 loader; POSIX mmap here) -----------------
 * kcb_gguf_open maps a llama- or qwen3-architecture GGUF file (Q4_K / Q6_K matrices, f32 norms) and fills `desc`
 * with pointers into the mapping, ready for kcb_model_create / kcb_decoder_create; the handle must stay open while
 * they upload (kcb_model_* also reads embedding rows from it afterwards).  No device needed. */
int kcb_gguf_open(const char* path, int max_ctx, void** gguf, kcb_model_desc* desc);
long long kcb_gguf_weight_bytes(void* gguf);   /* bytes of the matrices a token reads */
int kcb_gguf_close(void* gguf);
const char* kcb_gguf_last_error(void);

/* ---- graph-replayed decoder ---------------------------------------------------------------------------
 * The fast form of the decode loop (llm/llm_model.cpp:287-360; the reference's own CUDA comparison re-uses one
 * graph per token too, app/llm_bench.cpp:155-179): one CUDA graph captured at creation, replayed per token;
 * position and token live on the device; greedy next-token pick on the device; fp16 KV cache.
 * kcb_decoder_set_prompt places `n` forced tokens at positions start_pos.. (teacher forcing; after them the
 * decoder feeds back its own picks) and sets the position; kcb_decoder_run enqueues `steps` steps without
 * synchronising; kcb_decoder_read synchronises and copies the last step's logits (vocab floats), the picks
 * made at positions [0, n_history) and the current position.  Any output pointer may be NULL. */
int kcb_decoder_create(const kcb_model_desc* desc, void** decoder);
/* Tensor-parallel form over `world` (1..8) ranks, one process per GPU (the reference decodes on one device; its
 * row-chunked launches, llm/llm_kernels.cpp:281-288, are the split this extends across GPUs).  `desc` is the
 * whole model on every rank; rank r keeps heads, kv heads, FFN rows and vocabulary rows [r/world, (r+1)/world)
 * and the matching K windows of the attention-output and FFN-down matrices.  The two partial hidden vectors of
 * a layer are summed inside the following norm kernel straight out of the ranks' memories (ordinary loads over
 * NVLink, rank order, bounded waits), the greedy pick likewise over per-rank candidates.  shared[r] is rank r's
 * exchange area as mapped into this process (kcb_decoder_tp_shared_bytes bytes, peer-accessible, zero-filled
 * before any rank is created).  Ranks must replay in lockstep: same prompts, same step counts.
 * kcb_decoder_read returns vocab floats of which only this rank's rows are filled (others 0).
 * kcb_decoder_tp_timeouts: waits that gave up on this device since the library was loaded (0 = healthy). */
size_t kcb_decoder_tp_shared_bytes(const kcb_model_desc* desc);
int kcb_decoder_create_tp(const kcb_model_desc* desc, int rank, int world, void* const* shared, void** decoder);
unsigned kcb_decoder_tp_timeouts(void);
/* The same for the tensor-parallel decoder's exchanges: polls per wait (0 = default), and clearing the expiry count and
 * the "group dead" mark after which every exchange polls once and returns. */
int kcb_decoder_tp_set_poll_limit(unsigned polls);
int kcb_decoder_tp_reset(void);
int kcb_decoder_set_prompt(void* decoder, const int* tokens, int n, int start_pos);
/* Batched prompt pass: all n tokens through every layer together -- the reference's batched path in its
 * ggml backend (integrations/llama.cpp/ggml/src/ggml-kernelcore/ggml-kernelcore.cpp:548-589 mul_mat with per-256
 * activation slots, :502-522 fused norm, :663-697 attention over the fp16 cache) -- on the tensor-core matmuls.
 * Leaves the decoder where n single steps would: KV rows filled, logits and greedy pick of the last prompt token,
 * position start_pos + n; kcb_decoder_run then generates.  Returns after the pass has finished.  On a tensor-parallel
 * decoder every rank makes the same call; it needs each rank's share of the attention output and of the FFN to be a
 * whole number of 256-channel super-blocks and answers UnsupportedOperation otherwise (then feed the prompt through
 * kcb_decoder_set_prompt + kcb_decoder_run). */
int kcb_decoder_prefill(void* decoder, const int* tokens, int n, int start_pos);
int kcb_decoder_run(void* decoder, int steps);
/* A batch of independent sequences decoded in lockstep, on one GPU or tensor parallel under the same condition as the
 * batched prompt pass (the benchmark spec's batch-32 case; the reference's batched
 * path is its ggml backend with several tokens per graph, ggml-kernelcore.cpp:548-603): begin allocates one fp16 KV
 * cache per sequence; batch_prefill runs sequence `seq`'s prompt (all prompts the same length) and makes its first
 * pick; batch_run advances every sequence by `steps` greedy tokens, reading the weights once per step for the whole
 * batch; batch_read returns the last logits, the picks and the position of one sequence. */
int kcb_decoder_batch_begin(void* decoder, int n_sequences);
int kcb_decoder_batch_prefill(void* decoder, int seq, const int* tokens, int n);
int kcb_decoder_batch_run(void* decoder, int steps);
int kcb_decoder_batch_read(void* decoder, int seq, float* logits_host, int* history_host, int n_history, int* pos_host);
int kcb_decoder_sync(void* decoder);
int kcb_decoder_read(void* decoder, float* logits_host, int* history_host, int n_history, int* pos_host);
int kcb_decoder_info(void* decoder, int* launches_per_token, long long* weight_bytes);
void* kcb_decoder_stream(void* decoder);   /* the cudaStream_t the decoder runs on */
/* Test instrumentation (no counterpart in the reference; single-GPU decoders): after kcb_decoder_enable_trace every step
 * also keeps the int8 words of each activation vector it quantizes and the residual stream (hidden floats, as bit
 * patterns) after each of a layer's two additions, in the order the step runs -- layer 0's q|k|v input words, then per
 * layer the wo input words, the residual, the gate|up and down input words, the residual, the next q|k|v (after the last
 * layer: lm_head) input words; *words_per_step int32 words -- and kcb_decoder_read_trace copies the last step's to the
 * host (it waits for the stream).  The parity tests run the CPU restatement stage by stage on these inputs and count the
 * int8 values that rounded the other way (a value on a rounding boundary may, when a sum was taken in another order). */
int kcb_decoder_enable_trace(void* decoder, size_t* words_per_step);
int kcb_decoder_read_trace(void* decoder, int* words_host, size_t n_words);
int kcb_decoder_destroy(void* decoder);
const char* kcb_decoder_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
