/*
 * zen_cuda.h -- C-ABI of the B200 (sm_100a) backend for ZenInfer's block-quantised
 * GEMV/GEMM path.  Plain pointers and sizes only; no CUDA or C++ types, so the
 * reference's host code (or any FFI) can bind it without seeing a vendor header,
 * which is the same rule the reference's own GPU backends follow
 * (include/zen/hip_backend.h:8-13).
 *
 * Two groups of entry points:
 *
 *  1. HOST-POINTER calls.  These are the drop-in surface: one per function the
 *     reference's dispatch (src/quant.cpp) calls on a GPU backend.  `weights` is a
 *     host pointer to raw GGUF blocks (the loader's file mapping); the backend keeps
 *     a device copy keyed by (pointer, rows, columns, format) until it is released.
 *     `x` / `y` are caller-owned host fp32 buffers; a call returns after `y` is
 *     written.  Return 1 on success, 0 on failure.  There is no CPU fallback: 0 is
 *     an error, and zen_cuda_last_error() says why.
 *
 *  2. DEVICE-POINTER calls ("zen_cuda_dev_*").  Stream-ordered, no host
 *     synchronisation, activations stay in HBM between projections.  They replace
 *     the reference's per-call compute-pool hand-off (src/compute_pool.cpp:93-120)
 *     on this path, and are what its fused D3D12 submissions
 *     (include/zen/d3d12_backend.h:289-352) answer on that backend.
 *
 * Thread safety: any thread may call; calls are serialised on one backend mutex,
 * like the reference (src/backends/hip/hip_backend.hip:943).
 */
#ifndef ZEN_CUDA_H
#define ZEN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* GGML tensor type ids of the three formats on the path (GGUF tensor directory). */
enum { ZEN_CUDA_Q4_0 = 2, ZEN_CUDA_Q8_0 = 8, ZEN_CUDA_Q6_K = 14, ZEN_CUDA_Q4_K = 12, ZEN_CUDA_Q5_K = 13 };

/* How activations enter the integer dot products.
 *   ZEN_CUDA_ACT_INT8 : one int8 code per element, bit-identical to the reference's
 *                       quantise_acts_q8_0 (kernels/avx2.cpp:502-524); results match the
 *                       reference's ZEN_CPU_Q8_ACT=1 arithmetic.  Q8_0 only.
 *   ZEN_CUDA_ACT_FP32 : two int8 digits per element (error < scale/512); results match
 *                       the reference's fp32-activation kernels within 1e-3.  The only
 *                       mode for Q4_0 and Q6_K, whose reference kernels take fp32. */
enum { ZEN_CUDA_ACT_INT8 = 1, ZEN_CUDA_ACT_FP32 = 2 };

/* zen::hip::AdapterInfo, include/zen/hip_backend.h:16-23 */
typedef struct zen_cuda_adapter_info {
    char name[128];
    uint64_t dedicated_vram;
    uint64_t shared_memory;
    int sm_count;
    int warp_size;
    char arch[64]; /* "sm_100" */
} zen_cuda_adapter_info;

/* zen::hip::Stats, include/zen/hip_backend.h:25-41 */
typedef struct zen_cuda_stats {
    uint64_t dispatches;   /* kernels launched */
    uint64_t submits;      /* host-pointer calls completed */
    uint64_t batches;
    uint64_t upload_bytes; /* raw GGUF bytes uploaded */
    uint64_t weight_bytes; /* device bytes held by resident weights */
    uint64_t upload_us;
    uint64_t alloc_us;
    uint64_t stage_us;
    uint64_t repack_us;
    uint64_t transfer_us;
    uint64_t wait_us;
    uint64_t launch_us;
    uint64_t readback_us;
    uint64_t gpu_us;
    uint64_t fallbacks;    /* calls that returned 0 */
} zen_cuda_stats;

/* One matvec target of a batched submission; all tasks share the input.
 * zen::hip::GemvTask, include/zen/hip_backend.h:64-69 */
typedef struct zen_cuda_gemv_task {
    const uint8_t* weights;
    float* y;
    size_t rows;
    size_t columns;
} zen_cuda_gemv_task;

/* zen::d3d12::GemmTask, include/zen/d3d12_backend.h:118-122 */
typedef struct zen_cuda_gemm_task {
    const uint8_t* weights;
    float* y;
    size_t rows;
} zen_cuda_gemm_task;

#define ZEN_CUDA_MAX_BATCH 8 /* zen::hip::kMaxBatch, include/zen/hip_backend.h:70 */

/* ---- lifecycle: zen::hip::enabled/init/shutdown/info/stats, include/zen/hip_backend.h:46-50 */
int zen_cuda_enabled(void);  /* 1 when a usable device exists and ZEN_BACKEND does not name another backend */
int zen_cuda_init(void);     /* lazy, cached, thread-safe; a failure is latched until shutdown */
void zen_cuda_shutdown(void);
int zen_cuda_info(zen_cuda_adapter_info* out);
void zen_cuda_get_stats(zen_cuda_stats* out);
const char* zen_cuda_last_error(void); /* message of the most recent failed call on any thread */

/* ---- host-pointer calls ------------------------------------------------------------------- */

/* Process-wide activation mode for the Q8_0 host-pointer calls (default ZEN_CUDA_ACT_INT8;
 * also settable with ZEN_CUDA_Q8_ACT=int8|fp32 before init).  Mirrors the reference's
 * ZEN_CPU_Q8_ACT switch (src/quant.cpp:1088-1092). */
int zen_cuda_set_q8_act_mode(int mode);
int zen_cuda_get_q8_act_mode(void);

/* zen::hip::gemv_q8_0, include/zen/hip_backend.h:59-60 */
int zen_cuda_gemv_q8_0(const uint8_t* weights, const float* x, float* y, size_t rows, size_t columns);
/* zen::hip::gemm_q8_0, include/zen/hip_backend.h:61-62.  output is token-major [tokens][rows]. */
int zen_cuda_gemm_q8_0(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns);
/* zen::hip::gemv_q8_0_batch, include/zen/hip_backend.h:72 */
int zen_cuda_gemv_q8_0_batch(const float* x, const zen_cuda_gemv_task* tasks, size_t count);
/* zen::d3d12::gemm_q8_0_batch, include/zen/d3d12_backend.h:169 */
int zen_cuda_gemm_q8_0_batch(const float* x, const zen_cuda_gemm_task* tasks, size_t count, size_t tokens, size_t columns);
/* zen::d3d12::gemm_q6_k, include/zen/d3d12_backend.h:96-97 (tokens == 1 is the GEMV) */
int zen_cuda_gemm_q6_k(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns);
/* Q4_0 has no GPU entry point in the reference (its CPU generic route, src/quant.cpp:1135-1162,
 * is the only implementation); same contract as gemm_q6_k. */
int zen_cuda_gemm_q4_0(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns);
/* zen::d3d12::gemm_kquant, include/zen/d3d12_backend.h:75-77 (hook sites src/quant.cpp:970-976 for one token, :1619 for a
 * batch): raw Q4_K (q5 == 0) or Q5_K (q5 != 0) super-blocks, fp32 activations, columns a multiple of 256.  The device
 * pointer calls take these formats too (zen_cuda_dev_upload / zen_cuda_dev_gemv with ZEN_CUDA_Q4_K / ZEN_CUDA_Q5_K;
 * no fused input, accumulation or gather).  A first, untuned kernel. */
int zen_cuda_gemm_kquant(const uint8_t* weights, const float* input, float* output, size_t tokens, size_t rows, size_t columns, int q5);

/* zen::hip::rms_norm, include/zen/hip_backend.h:74-76 (device side hip_backend.hip:724-776): row-wise root-mean-square
 * normalisation, y[r][c] = x[r][c] * rsqrt(mean_c(x[r]^2) + epsilon) * weight[c].  Host buffers x, y [rows][columns],
 * weight [columns].  The sum of squares is taken in double, as the reference's CPU rms_norm does
 * (src/adapters/dense_transformer_runtime.cpp:117-125). */
int zen_cuda_rms_norm(const float* x, const float* weight, float* y, size_t rows, size_t columns, float epsilon);

/* zen::hip::gemv_q8_0_ffn, include/zen/hip_backend.h:78-83 (hook site src/quant.cpp:1553-1580, device side
 * hip_backend.hip:778-870): y = down * (silu(gate * x) * (up * x)) as one submission, the ffn_rows-wide activation staying
 * on the device.  gate, up: raw Q8_0 [ffn_rows][columns]; down: raw Q8_0 [out_rows][ffn_rows]; x [columns]; y [out_rows].
 * Two launches: gate and up share one; the down projection applies silu(g) * u as it loads its activations.
 * Activations enter as the backend's Q8_0 mode says (zen_cuda_set_q8_act_mode). */
int zen_cuda_gemv_q8_0_ffn(const uint8_t* gate, const uint8_t* up, const uint8_t* down, const float* x, float* y, size_t ffn_rows,
                           size_t columns, size_t out_rows);

/* Device layout of Q6_K tensors uploaded from now on (tensors already resident keep theirs; a launch takes tensors of one
 * layout).  on != 0 (the default; ZEN_CUDA_Q6K_CODES=0 changes it): the 6-bit codes are unpacked on upload to one int8
 * per weight (q - 32, element order), beside the group scales and super-block scales: 1.07 bytes per weight of device
 * memory and HBM traffic instead of the file's 0.82, and the decode kernel no longer rebuilds codes from ql and qh, which
 * bound it by instruction issue.
 * on == 0: the file's ql | qh | scales planes.  Results are the same bit for bit.  Returns the previous setting, -1 on
 * failure. */
int zen_cuda_set_q6k_codes(int on);

/* Which kernel the many-row products take (zen_cuda_gemm_q8_0 and its batch form from nine rows on, the
 * zen_cuda_dev_gemm_q8_0 entry points, and the Q4_0 / Q6_K / Q4_K / Q5_K products below).  on != 0 (the default; ZEN_CUDA_GEMM_GROUPS=0 changes it): weights and activations
 * as two int8 digits under one scale per 256 weights, so that a whole group accumulates on the tensor cores and the sums
 * are read back once per group: results within ~5e-5 of the reference's sums in either activation mode (its bar is 1e-3),
 * three to four times the speed.  The tensor's two-digit planes (2 bytes per weight of device memory) are built at its
 * first such product and kept until it is released.  Columns must be a multiple of 256 and the workspace of the size
 * zen_cuda_gemm_workspace_bytes reports; otherwise, and with on == 0, the per-block kernel runs: exactly the reference's
 * per-block integer sums, scaled block by block.  zen_cuda_dev_gemm_q8_0_noalloc always takes the per-block kernel.
 * Returns the previous setting, -1 on failure. */
int zen_cuda_set_gemm_groups(int on);

/* Residency budget of the pointer-keyed weights: kVRAMBudgetPercent, src/backends/hip/hip_backend.hip:50 and :459-476.
 * The tensors the host-pointer calls keep resident stay below the budget (80 % of the device's memory unless set here
 * or by ZEN_CUDA_VRAM_BUDGET_MB; bytes == 0 restores the default).  A tensor that would cross it evicts the WHOLE keyed
 * set first (the loader asks in the same order every run, so evicting a part would only churn); one that does not fit
 * the budget by itself makes the call return 0, as does a batch whose tensors do not fit together.  An eviction in the
 * middle of a batch is followed by resolving the batch's tensors again before anything is launched.  Tensors held
 * through zen_cuda_dev_upload belong to the caller: they count toward the bytes held and are never evicted. */
int zen_cuda_set_vram_budget(uint64_t bytes);
/* Any pointer may be null.  held_bytes counts keyed and caller-held tensors; tensors counts the keyed set. */
int zen_cuda_residency(uint64_t* budget_bytes, uint64_t* held_bytes, uint64_t* tensors, uint64_t* evictions);

/* zen::d3d12::release_q8_0_weights / release_kquant_weights, include/zen/d3d12_backend.h:80,88.
 * Call before unmapping or reusing a weight address; drops every resident shape at that address. */
void zen_cuda_release_weights(const uint8_t* weights);

/* The activation quantiser on its own (the reference's quantise_acts_q8_0, kernels/avx2.cpp:502-524;
 * shaders/quantize_acts.hlsl).  Host buffers: x [tokens][columns], codes [tokens][columns],
 * scales [tokens][columns/32]. */
int zen_cuda_quantize_acts(const float* x, int8_t* codes, float* scales, size_t tokens, size_t columns);

/* ---- device-pointer, stream-ordered calls -------------------------------------------------- */

typedef struct zen_cuda_weights zen_cuda_weights; /* opaque resident tensor */

/* Upload rows [first_row, first_row + nrows) of a raw GGUF tensor of `rows_total` x `columns`
 * (row sharding for multi-GPU reads only this byte range of the mapping).  The handle stays
 * valid until zen_cuda_dev_free or shutdown.  Not keyed by pointer. */
zen_cuda_weights* zen_cuda_dev_upload(int format, const uint8_t* weights, size_t rows_total, size_t columns,
                                      size_t first_row, size_t nrows);
void zen_cuda_dev_free(zen_cuda_weights* w);
size_t zen_cuda_dev_weight_bytes(const zen_cuda_weights* w); /* device bytes held */

/* y[i] = W[i] * x for up to ZEN_CUDA_MAX_BATCH tensors of the same format and column count
 * sharing x.  d_x: device fp32 [tokens][columns] (tokens <= 8); d_y[i]: device fp32
 * [tokens][rows_i].  Enqueued on `stream` (a cudaStream_t, or NULL for the backend's own
 * stream); returns without synchronising.  act_mode is ZEN_CUDA_ACT_*. */
int zen_cuda_dev_gemv(const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_x,
                      size_t tokens, int act_mode, void* stream);

/* zen_cuda_dev_gemv for Q8_0 tensors whose input is the SwiGLU hidden state: x = silu(gate) * up is formed while the
 * activations are loaded for quantisation, so the down projection needs no separate activation launch
 * (zen::quant::ffn_gemv / the D3D12 gemv_q8_0_ffn submission, src/quant.cpp:1566-1571; silu_mul,
 * src/adapters/dense_transformer_runtime.cpp:193-199).  d_gate, d_up: device fp32 [tokens][columns]. */
int zen_cuda_dev_gemv_swiglu(const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_gate, const float* d_up,
                             size_t tokens, int act_mode, void* stream);

/* zen_cuda_dev_gemv for Q8_0 tensors with the layer's small operators folded into the product launch (for Q4_0 and
 * Q6_K tensors only the warm_next field may be set, and it is ignored), which is what the
 * reference's fused D3D12 submissions do (ffn_residual_fused and LayerDecodeParams, include/zen/d3d12_backend.h:289-352,
 * zen::quant::ffn_residual_fused, src/quant.cpp:1566-1611):
 *   norm_weight != NULL : the input is RMSNorm(x) * norm_weight, eps = norm_eps (rms_norm, :117-125), formed per CTA in the
 *                         prologue; x itself is left untouched;
 *   gate != NULL        : the input is silu(gate) * x (as zen_cuda_dev_gemv_swiglu); not together with norm_weight;
 *   accumulate != 0     : y += W x instead of y = W x: with y the residual stream this is the layer's residual add;
 *   warm_next != NULL   : a hint, the resident Q8_0 tensor the stream's next product will read: once its own copies are
 *                         issued the launch asks L2 for the start of that tensor (up to 192 KB per CTA), so the next launch
 *                         does not begin with a DRAM round trip.  Honoured for launches of at most 32 MB of weights (a larger
 *                         one keeps HBM busy by itself).  Changes no result; any field combination is allowed.
 *   swiglu_pair != 0    : the launch holds exactly two tensors of equal shape, gate and up (w[0], w[1]); the two halves of
 *                         every CTA compute row r of both at the same time and d_y[0] receives silu(W0 x) * (W1 x), the
 *                         input of the down projection (silu_mul, src/adapters/dense_transformer_runtime.cpp:193-199);
 *                         d_y[1] is not written.  With norm_weight this is gate|up of a layer in one launch, no SwiGLU
 *                         launch after it.  Not with accumulate; not in a list item. */
typedef struct zen_cuda_gemv_fusion {
    const float* norm_weight;
    float norm_eps;
    int accumulate;
    const float* gate;
    const zen_cuda_weights* warm_next;
    int swiglu_pair;
} zen_cuda_gemv_fusion;
int zen_cuda_dev_gemv_fused(const zen_cuda_weights* const* w, float* const* d_y, size_t count, const float* d_x, size_t tokens, int act_mode,
                            const zen_cuda_gemv_fusion* fusion, void* stream);

/* Several batch-1 Q8_0 products in ONE persistent launch: what the reference's fused D3D12 submissions do for a layer's
 * chain of matvecs (ffn_residual_fused: o, residual, norm, gate|up, SwiGLU, down, residual in one command list, and
 * layer_decode_pipeline, include/zen/d3d12_backend.h:289-352, zen::quant::ffn_residual_fused src/quant.cpp:1566-1611).
 * An item is one zen_cuda_dev_gemv_fused product (up to ZEN_CUDA_MAX_BATCH tensors sharing d_x, one token); the items
 * run in order, the weight stream never pauses between them, and every result is bit-identical to the same products
 * launched one by one.
 *   - depends_on_earlier_items != 0: the item's input (d_x, gate) or accumulated output is written by earlier items of
 *     the same list; its arithmetic starts once all of them are complete.  Leave it 0 for items that only read what
 *     was complete before the launch (independent tensors sharing an input, the bench's weight copies): hazards
 *     between such items are the caller's business.
 *   - fusion: as zen_cuda_dev_gemv_fused (warm_next is ignored: the list streams ahead by itself).
 *   - The list is built once (the items are copied to the device) and launched any number of times, like a graph; one
 *     list must not be in flight twice at the same time.  Pointers inside must stay valid while it exists.
 *   - The launch uses one CTA per SM and relies on all of them being resident together; waits are bounded like every
 *     device-side wait here (zen_cuda_dev_check code 9 when an item's input did not arrive). */
typedef struct zen_cuda_gemv_list zen_cuda_gemv_list;
typedef struct zen_cuda_gemv_list_item {
    const zen_cuda_weights* const* w;
    float* const* d_y;
    size_t count;
    const float* d_x;
    zen_cuda_gemv_fusion fusion;
    int depends_on_earlier_items;
} zen_cuda_gemv_list_item;
zen_cuda_gemv_list* zen_cuda_gemv_list_create(const zen_cuda_gemv_list_item* items, size_t count, int act_mode);
void zen_cuda_gemv_list_destroy(zen_cuda_gemv_list* list);
uint64_t zen_cuda_gemv_list_bytes(const zen_cuda_gemv_list* list); /* raw GGUF bytes + fp32 inputs and outputs of all items */
int zen_cuda_dev_gemv_list(const zen_cuda_gemv_list* list, void* stream);

/* Prefill product on the tensor cores (Q8_0, int8 activations): d_out[i] = d_x * W[i]^T, token-major
 * [tokens][rows_i].  d_x: device fp32 [tokens][columns]; `workspace` is device scratch of at least
 * zen_cuda_gemm_workspace_bytes(tokens, columns) bytes that must stay untouched until the work has run (it
 * receives the quantised activations: the reference's quantize_acts step, shaders/quantize_acts.hlsl, then
 * zen::d3d12::gemm_q8_0_batch, include/zen/d3d12_backend.h:169).  Stream-ordered, no synchronisation. */
size_t zen_cuda_gemm_workspace_bytes(size_t tokens, size_t columns);
int zen_cuda_dev_gemm_q8_0(const zen_cuda_weights* const* w, float* const* d_out, size_t count, const float* d_x,
                           size_t tokens, void* workspace, size_t workspace_bytes, void* stream);
/* The same product with the activation mode named.  ZEN_CUDA_ACT_FP32 is the tensor-core counterpart of the reference's
 * default prefill kernel, which takes fp32 activations (src/quant.cpp:1667-1680 -> gemm_q8_0_kblk_avx2,
 * kernels/avx2.cpp:878-1248): every activation enters as two int8 digits, a block costs two MMAs, and results stay
 * within ~1e-5 of the fp32-activation product (the bar is 1e-3).  Its workspace also holds the second digit:
 * zen_cuda_gemm_workspace_bytes_act(tokens, columns, act_mode).  The host-pointer calls (zen_cuda_gemm_q8_0,
 * zen_cuda_gemm_q8_0_batch) take this path for more than eight tokens in either mode. */
size_t zen_cuda_gemm_workspace_bytes_act(size_t tokens, size_t columns, int act_mode);
int zen_cuda_dev_gemm_q8_0_act(const zen_cuda_weights* const* w, float* const* d_out, size_t count, const float* d_x,
                               size_t tokens, int act_mode, void* workspace, size_t workspace_bytes, void* stream);

/* Q6_K product for two or more activation rows on the tensor cores (the batched lm_head of config 3, and the reference's
 * batched Q6_K product gemm_q6k_kblk_avx2, kernels/avx2.cpp:1762-1770, GPU entry zen::d3d12::gemm_q6_k,
 * include/zen/d3d12_backend.h:169): fp32-equivalent activations (two int8 digits), out [tokens][rows] fp32.  The tensor
 * must be resident with its codes unpacked (the default layout, zen_cuda_set_q6k_codes).  `workspace` is device memory of
 * at least zen_cuda_gemm_q6_k_workspace_bytes(tokens, columns), untouched until the stream has run the work.  Up to
 * sixteen rows go through tiles of 32 columns (a token is two columns, one per parity of its 16-weight groups), more
 * through the prefill GEMM's 128.  The host-pointer call zen_cuda_gemm_q6_k takes this path by itself from seven rows
 * on; below that the decode kernel is faster.  With the group-scale kernel enabled (zen_cuda_set_gemm_groups) the product
 * runs over the tensor's cached two-digit planes instead. */
size_t zen_cuda_gemm_q6_k_workspace_bytes(size_t tokens, size_t columns);
int zen_cuda_dev_gemm_q6_k(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* workspace,
                           size_t workspace_bytes, void* stream);

/* Q4_0 times many activation rows on the tensor cores (the reference multiplies Q4_0 through its generic fp32 route,
 * src/quant.cpp:1135-1162, and has no GPU entry for the format): the nibbles are widened to int8 codes n - 8 in the
 * workspace, which with the tensor's f16 block scales is a Q8_0 tensor, then the Q8_0 GEMM runs with fp32-equivalent
 * activations.  `workspace`: device memory of at least zen_cuda_gemm_q4_0_workspace_bytes(tokens, rows, columns) --
 * rows x columns bytes of codes plus the GEMM's own workspace -- untouched until the stream has run the work; columns
 * must be a multiple of 128.  The host-pointer call zen_cuda_gemm_q4_0 takes this path by itself from nine rows on.  With
 * whole 256-weight groups and the group-scale kernel enabled (zen_cuda_set_gemm_groups) the product runs over the tensor's
 * cached two-digit planes instead and nothing is widened per call. */
size_t zen_cuda_gemm_q4_0_workspace_bytes(size_t tokens, size_t rows, size_t columns);
int zen_cuda_dev_gemm_q4_0(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* workspace,
                           size_t workspace_bytes, void* stream);

/* Q4_K / Q5_K times many activation rows on the tensor cores (the reference's batched K-quant products gemm_q4k_kblk_avx2 /
 * gemm_q5k_kblk_avx2, kernels/avx2.cpp:1605-1620; GPU entry zen::d3d12::gemm_kquant, include/zen/d3d12_backend.h:75): the
 * 4- and 5-bit codes are widened to int8 in the workspace together with the fp32 factors of every 32-weight sub-block
 * (d * sc and dmin * m, as the reference forms them), then the GEMM runs with fp32-equivalent activations and subtracts
 * the minimum term in its epilogue.  `workspace`: at least zen_cuda_gemm_kquant_workspace_bytes(tokens, rows, columns) of
 * device memory, untouched until the stream has run the work.  The host-pointer call zen_cuda_gemm_kquant takes this path
 * by itself from nine rows on.  With the group-scale kernel enabled (zen_cuda_set_gemm_groups) the product runs over the
 * tensor's cached two-digit planes instead and nothing is widened per call. */
size_t zen_cuda_gemm_kquant_workspace_bytes(size_t tokens, size_t rows, size_t columns);
int zen_cuda_dev_gemm_kquant(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* workspace,
                             size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  The same prefill product as zen_cuda_dev_gemm_q8_0 for ONE tensor, for callers
 * that may not allocate device memory at the time of the call: a plug-in living inside a host runtime that owns all of
 * HBM (weights, KV cache and arenas were sized at start-up and nothing is left to ask for), or a serving loop that can
 * not afford the device-wide synchronisation an allocation or a free implies.  Such callers have no workspace to hand
 * in, so this entry point keeps the quantised activations in a fixed scratch array that is part of the library image
 * (ZEN_CUDA_NOALLOC_SCRATCH_BYTES of HBM on every GPU that loads the library, held until the process exits).  It calls
 * no cudaMalloc / cudaFree and no allocating library routine, and it does not initialise the backend: the tensor must
 * already be resident (zen_cuda_dev_upload), which is also what makes the backend ready.
 *   - tokens * columns must not exceed ZEN_CUDA_NOALLOC_MAX_ACT_ELEMENTS, and the quantised activations with their
 *     scale rows (zen_cuda_gemm_workspace_bytes) must fit ZEN_CUDA_NOALLOC_SCRATCH_BYTES; larger requests return 0
 *     with a message.
 *   - What CUDA itself allocates lazily on first use -- the array when its address is first looked up, the code of the
 *     kernels, the GEMM's shared-memory opt-in -- is done when the backend starts (zen_cuda_init or the first upload,
 *     where allocating is allowed), once per device and with that device current, so this call finds all of it in
 *     place.  Start the backend before any stream capture begins.
 *   - Every call uses the same array and finds the previous call's bytes in it (the part a call reads is rewritten,
 *     and its scale area is cleared, first).  Two calls whose GPU work overlaps (different streams, or different
 *     threads without ordering) race on it: order them on one stream or with events.
 * d_x: device fp32 [tokens][columns]; d_out: device fp32 [tokens][rows]; stream: a cudaStream_t or NULL. */
#define ZEN_CUDA_NOALLOC_MAX_ACT_ELEMENTS 2097152u /* e.g. 512 tokens x 4096 columns */
#define ZEN_CUDA_NOALLOC_SCRATCH_BYTES (2097152u + 262144u)
int zen_cuda_dev_gemm_q8_0_noalloc(const zen_cuda_weights* w, float* d_out, const float* d_x, size_t tokens, void* stream);

/* Device quantiser: d_x [tokens][columns] fp32 -> d_codes int8, d_scales fp32 [tokens][columns/32]. */
int zen_cuda_dev_quantize_acts(const float* d_x, int8_t* d_codes, float* d_scales, size_t tokens, size_t columns, void* stream);

/* ---- row-sharded products across GPUs: the output all-gather fused into the decode kernel ------------------------
 * No counterpart in the reference, which drives one device; the row cut is its worker cut (ComputePool::parallel_for,
 * src/compute_pool.cpp:104-106).  One process per GPU.  Every rank allocates a gather region, the ranks exchange the
 * 64-byte IPC handles through whatever channel the host has (the tests and the benchmark use torch.distributed), open
 * each other's regions and bind them into a gather object.  zen_cuda_dev_gemv_gather then runs the rank's shard of the
 * product and stores every output into the rank's slot of EVERY rank's region from inside the product kernel (peer
 * stores over NVLink); the grid's last CTA publishes the launch to all ranks.  A later launch on any rank that
 * consumes the gathered vector waits on the device, with a time limit of about a second, until all ranks have published
 * it; on expiry the error word is set (zen_cuda_dev_check) and nothing hangs.
 *   - All ranks must enqueue the same sequence of gather launches on a gather object.
 *   - A slot holds [tokens][sum of the launch's rows] floats and must fit slot_floats.
 *   - The gathered vector of launch n, [world][slot_floats], stays intact until launch n+2 starts writing.
 *   - Before zen_cuda_gather_destroy / zen_cuda_ipc_free the host must make sure (a barrier after a stream
 *     synchronise) that no rank still has a launch in flight that writes here. */
#define ZEN_CUDA_MAX_PEERS 8
#define ZEN_CUDA_IPC_HANDLE_BYTES 64
typedef struct zen_cuda_gather zen_cuda_gather;
size_t zen_cuda_gather_region_bytes(size_t world, size_t slot_floats);
/* cudaMalloc'd, zero-filled device memory whose IPC handle is written to handle_out; NULL on failure. */
void* zen_cuda_ipc_alloc(size_t bytes, unsigned char handle_out[ZEN_CUDA_IPC_HANDLE_BYTES]);
void* zen_cuda_ipc_open(const unsigned char handle[ZEN_CUDA_IPC_HANDLE_BYTES]); /* a peer's region, mapped here */
void zen_cuda_ipc_close(void* peer_region);
void zen_cuda_ipc_free(void* own_region);
/* regions[r] = rank r's region as addressed from this process (regions[rank] = the own allocation). */
zen_cuda_gather* zen_cuda_gather_create(size_t world, size_t rank, size_t slot_floats, void* const* regions);
void zen_cuda_gather_destroy(zen_cuda_gather* g);
/* The shard product of zen_cuda_dev_gemv with the gather fused in.  d_x == NULL: the input is the vector gathered by
 * the previous launch on this object (columns must equal world * slot_floats, tokens 1).  d_y may be NULL (or hold
 * NULL entries) when only the gathered copy is wanted. */
int zen_cuda_dev_gemv_gather(zen_cuda_gather* g, const zen_cuda_weights* const* w, float* const* d_y, size_t count,
                             const float* d_x, size_t tokens, int act_mode, void* stream);
/* Waits (on the device, bounded) until the latest launch of every rank has landed here and copies the gathered
 * vector, [world][slot_floats] floats, to d_out (NULL: wait only). */
int zen_cuda_dev_gather_fetch(zen_cuda_gather* g, float* d_out, void* stream);
/* A plain all-gather of device vectors over a gather object's regions (peer stores over NVLink, flags, a bounded device
 * wait; one launch, no collective library): rank r's d_piece (count floats, a multiple of 4, at most slot_floats, 16-byte
 * aligned) lands in every rank's d_whole at [r * count, (r + 1) * count); d_piece may be this rank's slice of d_whole.
 * For the vectors between the row-sharded projections of a decode step (attention output, residual stream, SwiGLU
 * activation, logits).  All ranks enqueue the same sequence of these calls on the object; an object used here must not
 * also be used by zen_cuda_dev_gemv_gather.  No counterpart in the reference (one device). */
int zen_cuda_dev_allgather(zen_cuda_gather* g, const float* d_piece, size_t count, float* d_whole, void* stream);
/* The all-reduce that goes with a projection cut by columns: d_inout[i] += sum over ranks of that rank's d_partial[i]
 * (count floats, same rules as above), added in rank order on every rank, so all ranks end with identical values.
 * Shares the object's launch numbering with zen_cuda_dev_allgather: the two may alternate on one object. */
int zen_cuda_dev_allreduce_add(zen_cuda_gather* g, const float* d_partial, size_t count, float* d_inout, void* stream);

/* Greedy token pick on the device: for every token row, the index of the first maximum among the finite logits,
 * -1 when the row has none.  The greedy branch of the reference's sampler (sample_logits,
 * src/adapters/dense_transformer_runtime.cpp:391-418): the lowest index wins ties, non-finite logits never win.
 * A row may be given in up to ZEN_CUDA_MAX_PEERS segments, which is the layout a row-sharded lm_head leaves behind
 * ([rank][token][shard rows], zen_cuda_dev_gather_fetch): segment i covers row entries
 * [first_index, first_index + len) and token t of it starts at base + t * token_stride.  d_pick: device int64
 * [tokens].  Stream-ordered, no synchronisation. */
typedef struct zen_cuda_pick_segment {
    const float* base;
    uint32_t len;
    uint32_t first_index;
    uint32_t token_stride;
    uint32_t reserved;
} zen_cuda_pick_segment;
int zen_cuda_dev_greedy_pick(const zen_cuda_pick_segment* segments, size_t count, size_t tokens, int64_t* d_pick, void* stream);

/* Temperature / top-k / top-p sampling on the device: the non-greedy branch of the reference's sampler
 * (sampling_distribution + sample_distribution, src/adapters/dense_transformer_runtime.cpp:349-390).  Among the finite
 * logits the top_k highest are kept (ties at the cut go to the lowest ids), p_i = exp((v_i - max) / temperature) is
 * normalised over them in double, the top-p cut keeps the shortest prefix (by descending probability) whose cumulative
 * probability reaches top_p (at least one token), and the token is drawn from the kept ones IN TOKEN-ID ORDER as the
 * first whose cumulative probability reaches u -- the walk std::discrete_distribution does over the reference's
 * id-indexed probability vector; u is a uniform number in [0, 1) from the caller's generator, which stays on the host.
 *   temperature > 0 (use zen_cuda_dev_greedy_pick otherwise); top_p >= 1 or <= 0: no top-p cut.
 *   At most ZEN_CUDA_SAMPLE_MAX_CANDIDATES tokens are considered: with top_k == 0 or larger the tail beyond the 1024
 *   most likely tokens is dropped, and *d_truncated (optional) is set when the top-p nucleus did not fit into them.
 *   d_pick: device int64, -1 when no logit is finite.  d_kept_ids / d_kept_probs (optional, room for
 *   ZEN_CUDA_SAMPLE_MAX_CANDIDATES entries) receive the kept ids in ascending order and their probabilities (sum 1),
 *   d_kept_count (optional) their number: a host that wants to draw itself reads these instead.
 * Logit bias and allowed-token lists of the reference's options are applied by the caller to the logits beforehand. */
#define ZEN_CUDA_SAMPLE_MAX_CANDIDATES 1024
int zen_cuda_dev_sample(const float* d_logits, size_t n, float temperature, uint32_t top_k, float top_p, double u, int64_t* d_pick,
                        int32_t* d_kept_ids, double* d_kept_probs, int32_t* d_kept_count, int32_t* d_truncated, void* stream);

/* ---- the decode-step operators between the projections (device pointers, stream-ordered, no synchronisation) -----
 * With these a whole token step of a dense Llama-style layer stays in HBM on one stream.  They answer the reference's
 * host loop in DenseTransformerRuntime::forward (src/adapters/dense_transformer_runtime.cpp:3670-4600) and the
 * per-operator submissions its D3D12 backend offers for the same steps (include/zen/d3d12_backend.h:176 rms_norm,
 * :192 rope_apply, :231 kv_cache_append, :247 attention_block, :370 silu_mul).  The position of the token in flight
 * is read from device memory (d_pos), so a captured launch sequence can be replayed for every step. */

/* d_out[columns] = row *d_token of a resident Q8_0 tensor, decoded to fp32 (the embedding fetch,
 * src/adapters/dense_transformer_runtime.cpp:3692 over src/quant.cpp:410-416).  d_token: device int64. */
int zen_cuda_dev_embed_q8_0(const zen_cuda_weights* w, const int64_t* d_token, float* d_out, void* stream);
/* Per row of n floats: if d_delta is given, x += delta in place first (the residual add); then, if d_weight is given,
 * y = x * inv * weight with inv = 1 / sqrt(float(sum x^2 / n) + eps), the sum taken in double
 * (rms_norm, src/adapters/dense_transformer_runtime.cpp:117-125). */
int zen_cuda_dev_rms_norm(float* d_x, const float* d_delta, const float* d_weight, float* d_y, size_t n, size_t rows, float eps, void* stream);
/* Rotary embedding of q [heads][head_dim] and k [kv_heads][head_dim] in place with row *d_pos of the HOST-BUILT tables
 * d_cos / d_sin [positions][pairs] (the table contract of rope_table, src/adapters/dense_transformer_runtime.cpp:264-276:
 * the device computes no angle), pairs (x[2i], x[2i+1]) when adjacent != 0, else (x[i], x[i+pairs]); then k and v are
 * appended to the layer's fp32 caches [max_positions][kv_heads * head_dim] at *d_pos. */
int zen_cuda_dev_rope_kv_append(float* d_q, float* d_k, const float* d_v, const float* d_cos, const float* d_sin, const int* d_pos,
                                size_t heads, size_t kv_heads, size_t head_dim, size_t pairs, int adjacent, float* d_k_cache, float* d_v_cache,
                                size_t max_positions, void* stream);
/* Grouped-query attention of one new token over positions [first, *d_pos] of the layer's caches, first = 0 or the
 * sliding-window start; query head h reads kv head h / (heads / kv_heads)
 * (src/adapters/dense_transformer_runtime.cpp:4284-4337).  scale 0 means 1 / sqrt(head_dim).  d_out [heads][head_dim]. */
int zen_cuda_dev_attention(const float* d_q, const float* d_k_cache, const float* d_v_cache, const int* d_pos, float* d_out, size_t heads,
                           size_t kv_heads, size_t head_dim, float scale, size_t window, size_t max_positions, void* stream);
/* The attention block of one new token in one launch (zen::d3d12::attention_block, include/zen/d3d12_backend.h:247): q, k, v
 * are the raw projections; the adjacent-pair rotary embedding (row *d_pos of the host-built tables, `pairs` pairs per head)
 * is applied to q and k inside the kernel, k and v are appended to the caches at *d_pos, and the attention of
 * zen_cuda_dev_attention runs over [first, *d_pos].  d_q and d_k are left untouched. */
int zen_cuda_dev_attention_block(const float* d_q, const float* d_k, const float* d_v, const float* d_cos, const float* d_sin, size_t pairs,
                                 const int* d_pos, float* d_k_cache, float* d_v_cache, float* d_out, size_t heads, size_t kv_heads, size_t head_dim,
                                 float scale, size_t window, size_t max_positions, void* stream);
/* ---- the same operators over a block of `tokens` new tokens at positions *d_pos .. *d_pos + tokens - 1 (prefill and
 * speculative verify: DenseTransformerRuntime::forward_batch, src/adapters/dense_transformer_runtime.cpp:2296-3664; the
 * D3D12 counterparts are rope_apply_prefill, kv_cache_append_batched and the flash-attention submissions,
 * include/zen/d3d12_backend.h:207,235).  Buffers are token-major: q [tokens][heads * head_dim] and so on; the projections
 * between them are zen_cuda_dev_gemm_q8_0, the norms zen_cuda_dev_rms_norm with rows = tokens. */
int zen_cuda_dev_embed_rows_q8_0(const zen_cuda_weights* w, const int64_t* d_tokens, size_t tokens, float* d_out, void* stream);
int zen_cuda_dev_rope_kv_append_rows(float* d_q, float* d_k, const float* d_v, size_t tokens, const float* d_cos, const float* d_sin, const int* d_pos,
                                     size_t heads, size_t kv_heads, size_t head_dim, size_t pairs, int adjacent, float* d_k_cache, float* d_v_cache,
                                     size_t max_positions, void* stream);
/* Causal attention: token t attends positions [first, *d_pos + t] of the caches (which already hold the block's keys
 * and values).  head_dim 64, 128 or 256. */
int zen_cuda_dev_attention_prefill(const float* d_q, const float* d_k_cache, const float* d_v_cache, const int* d_pos, float* d_out, size_t tokens,
                                   size_t heads, size_t kv_heads, size_t head_dim, float scale, size_t window, size_t max_positions, void* stream);
/* d_out = silu(gate) * up (silu_mul, src/adapters/dense_transformer_runtime.cpp:193-199). */
int zen_cuda_dev_silu_mul(const float* d_gate, const float* d_up, float* d_out, size_t count, void* stream);
/* *d_pos += delta, in stream order (a step's last launch). */
int zen_cuda_dev_advance_position(int* d_pos, int delta, void* stream);

/* The device-side error channel.  Synchronises `stream` (NULL: the backend's own), then reads and clears the error word
 * the kernels set.  Returns
 *    0      nothing to report;
 *    1..4   a bounded wait inside a product kernel gave up (weight stage full / empty, drain at exit, tensor memory);
 *    5      a peer GPU did not publish its outputs within the wait budget;
 *    6, 7   a token id outside the embedding table / a position outside the KV cache (the kernel wrote zeros);
 *    8      a non-finite value met in attention;
 *    9      a work-list item's input was not produced within the wait budget;
 *    < 0    the synchronise itself or an earlier launch failed in the CUDA runtime (-(cudaError_t) - 1), or the backend
 *           is not initialised (-1): zen_cuda_last_error() has the text.
 * The kernels never spin for ever: every device-side wait is bounded by the wait budget below, after which the kernel
 * sets the word and returns, and the context stays usable.  (The reference reports GPU failures as a `false` return of
 * the submitting call, src/backends/hip/hip_backend.hip:947-950; stream-ordered calls have no such moment.) */
int zen_cuda_dev_check(void* stream);
const char* zen_cuda_error_name(int code); /* a static string for a zen_cuda_dev_check code */
/* The wait budget of every bounded device-side wait, in milliseconds of the top SM clock (default about one second;
 * 0 restores the default; ZEN_CUDA_WAIT_MS sets it at start-up).  Drains the backend's own stream first; kernels
 * already enqueued on other streams may see either value.  No counterpart in the reference. */
int zen_cuda_set_wait_budget_ms(unsigned milliseconds);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ZEN_CUDA_H */
