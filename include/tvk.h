/*
 * tvk.h — C-ABI of the B200-native runtime and kernels that sit underneath the
 * torchvulkan ATen operator layer.
 *
 * Everything the reference keeps in src/vulkan (device contexts, allocator and
 * buffer cache, copies, the shader manager's dispatchShader) and in src/shaders
 * (the Slang kernels) is reached through the functions declared here.  The
 * signatures carry plain pointers and sizes only: no torch types, no C++ types,
 * no exceptions.  All pointers are device pointers owned by the caller unless a
 * parameter is documented as a host pointer.  No kernel entry point allocates:
 * outputs and scratch are passed in; scratch sizes come from the
 * *_workspace_size queries.
 *
 * Every function returns a tvk_status (0 = success).  On failure a thread-local
 * message is available from tvk_last_error().  Nothing here aborts, throws or
 * traps the device.  Any device-side wait is bounded; a wait that runs out is
 * reported as TVK_ERR_TIMEOUT by tvk_check_device_status().
 *
 * `stream` arguments are cudaStream_t handles passed as void*; NULL selects the
 * CUDA default stream of the current device.
 */
#ifndef TVK_H_
#define TVK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TVK_API __attribute__((visibility("default")))

typedef enum tvk_status {
    TVK_OK = 0,
    TVK_ERR_INVALID = 1,      /* bad argument (shape, stride, null pointer, dtype)          */
    TVK_ERR_UNSUPPORTED = 2,  /* valid request this build has no kernel for                 */
    TVK_ERR_OOM = 3,          /* device allocation failed after the cache was released      */
    TVK_ERR_CUDA = 4,         /* a CUDA runtime/driver call failed                          */
    TVK_ERR_TIMEOUT = 5,      /* a bounded device-side wait ran out                         */
    TVK_ERR_BAD_FORK = 6,     /* used in a forked child of an initialised parent            */
    TVK_ERR_NO_DEVICE = 7     /* no CUDA device / driver                                    */
} tvk_status;

typedef enum tvk_dtype {
    TVK_F32 = 0,
    TVK_F16 = 1,
    TVK_BF16 = 2,
    TVK_I64 = 3,
    TVK_I32 = 4,
    TVK_U8 = 5,   /* also bool */
    TVK_F64 = 6   /* copies/fills only */
} tvk_dtype;

#define TVK_MAX_DIMS 8

/* Last error message of the calling thread ("" if none). */
TVK_API const char* tvk_last_error(void);
/* Library version string, and the SM architecture the kernels were built for. */
TVK_API const char* tvk_version(void);

/* ------------------------------------------------------------------------- *
 * Runtime: devices, streams, memory.
 * Replaces VulkanContext / DeviceContext (src/vulkan/vulkan_context.h:9-33,
 * src/vulkan/device_context.h:24-88).
 * ------------------------------------------------------------------------- */

typedef struct tvk_device_props {
    char name[256];
    uint64_t total_memory;
    uint32_t vendor_id;       /* PCI vendor id (0x10DE)                                   */
    uint32_t device_id;       /* PCI device id                                            */
    int32_t cc_major, cc_minor;
    int32_t driver_version;   /* cudaDriverGetVersion                                     */
    int32_t runtime_version;  /* cudaRuntimeGetVersion                                    */
    int32_t sm_count;
    int32_t warp_size;        /* the reference's "subgroup_size"                          */
    int32_t l2_bytes;
    int32_t max_smem_per_block;
} tvk_device_props;

/* VulkanContext::getDeviceCount (src/vulkan/vulkan_context.h:16). 0 devices is not an error. */
TVK_API int tvk_device_count(int* count);
/* VulkanContext::IsInitialized / Instance() lazy init (src/vulkan/vulkan_context.cpp:124-151). */
TVK_API int tvk_is_initialized(void);
TVK_API int tvk_init(void);
/* VulkanContext::IsInBadFork (src/vulkan/vulkan_context.cpp:119-133). */
TVK_API int tvk_is_in_bad_fork(void);
/* VulkanContext::CurrentDevice / SetCurrentDevice: per-thread (src/vulkan/vulkan_context.cpp:36). */
TVK_API int tvk_set_device(int dev);
TVK_API int tvk_get_device(int* dev);
TVK_API int tvk_get_device_props(int dev, tvk_device_props* out);
/* The in-order compute stream of a device (replaces the deferred op list + DAG dispatcher,
 * src/vulkan/shader.cpp:100-121, src/vulkan/dispatch.cpp:65-169). */
TVK_API int tvk_get_stream(int dev, void** stream);
/* DeviceContext::flush (src/vulkan/device_context.cpp:29-51): wait for all work on the device. */
TVK_API int tvk_synchronize(int dev);
/* Reads (and clears) the device-side status word written by kernels whose bounded waits ran
 * out. Returns TVK_OK or TVK_ERR_TIMEOUT. Synchronises the device. */
TVK_API int tvk_check_device_status(int dev);

typedef struct tvk_mem_stats {
    uint64_t allocated_bytes;       /* live bytes handed to callers (rounded sizes)       */
    uint64_t peak_allocated_bytes;
    uint64_t reserved_bytes;        /* live + cached                                      */
    uint64_t cached_bytes;
    uint64_t total_allocated_bytes; /* cumulative                                         */
    uint64_t total_freed_bytes;     /* cumulative                                         */
    uint64_t num_device_mallocs;    /* calls that reached the raw device allocator        */
    uint64_t num_cache_hits;
    uint64_t num_oom_retries;       /* times the cache was emptied to satisfy a request   */
} tvk_mem_stats;

/* Size-class rounding of the caching allocator: quarter-octave steps, 256 B minimum
 * (same classes as VulkanCache::roundBufferSize, src/vulkan/cache.cpp:78-87). */
TVK_API uint64_t tvk_round_size(uint64_t bytes);
/* VulkanAllocator::allocate / deleter (src/vulkan/allocator.cpp:59-83, 171-201): cache hit,
 * else device malloc, else release the cache and retry, else TVK_ERR_OOM. Frees are
 * stream-ordered on the device's compute stream. bytes == 0 yields *ptr == NULL. */
TVK_API int tvk_malloc(int dev, uint64_t bytes, void** ptr);
TVK_API int tvk_free(int dev, void* ptr);
/* DeviceContext::releaseCachedBuffers (src/vulkan/device_context.h:80-83). */
TVK_API int tvk_empty_cache(int dev);
/* DeviceContext::memoryFree/memoryTotal (src/vulkan/device_context.cpp:53-73). */
TVK_API int tvk_mem_info(int dev, uint64_t* free_bytes, uint64_t* total_bytes);
/* Atomic counters of src/vulkan/device_context.h:64-68 / getDeviceStats (allocator.cpp:21-37). */
TVK_API int tvk_mem_get_stats(int dev, tvk_mem_stats* out);
TVK_API int tvk_mem_reset_peak(int dev);
/* Pinned host staging memory (src/vulkan/memory.cpp:7-60 host-visible variants). */
TVK_API int tvk_host_alloc(uint64_t bytes, void** host_ptr);
TVK_API int tvk_host_free(void* host_ptr);

/* Test hooks: replace the raw device allocator underneath the cache so the allocator's
 * ladder can be exercised on a machine without a GPU. Pass NULLs to restore cudaMalloc. */
typedef int (*tvk_raw_alloc_fn)(void** ptr, uint64_t bytes);
typedef int (*tvk_raw_free_fn)(void* ptr);
TVK_API int tvk_debug_set_raw_allocator(tvk_raw_alloc_fn a, tvk_raw_free_fn f, int fake_device_count);
/* Test hook for the timeout convention: launches a one-thread kernel that polls a flag nothing ever sets, gives up
 * after `polls` tries (100 ns apart, polls <= 10^6, i.e. at most a tenth of a second) and records the time-out in the
 * device status word exactly as the waits inside the GEMM, convolution and attention kernels do. The next
 * tvk_check_device_status(dev) answers TVK_ERR_TIMEOUT, and the device stays usable. */
TVK_API int tvk_debug_bounded_wait(int dev, int polls, void* stream);

/* Copies (VulkanAllocator::copy_host_to_device / copy_device_to_host / copy_device_to_device,
 * src/vulkan/allocator.cpp:90-162). h2d/d2d are asynchronous on the device's compute stream;
 * d2h returns after the bytes have landed in host memory (the reference flushes there). */
TVK_API int tvk_memcpy_h2d(int dev, void* dst, const void* host_src, uint64_t bytes);
TVK_API int tvk_memcpy_d2h(int dev, void* host_dst, const void* src, uint64_t bytes);
TVK_API int tvk_memcpy_d2d(int dev, void* dst, const void* src, uint64_t bytes);
/* Cross-device copy; the reference bounces through the host (allocator.cpp:143-161), here it
 * is a peer copy over NVLink. */
TVK_API int tvk_memcpy_peer(int dst_dev, void* dst, int src_dev, const void* src, uint64_t bytes);
/* Device-to-device copy on a stream of the caller's (copy_device_to_device, src/vulkan/allocator.cpp:143-161, without
 * the library's own stream): dst or src may be another device's memory mapped into this process (tvk_ipc_open, or a
 * peer-enabled device), in which case the bytes travel over NVLink on a copy engine and occupy no SM. */
TVK_API int tvk_memcpy_async(void* dst, const void* src, uint64_t bytes, void* stream);

/* Device that owns a pointer handed out by tvk_malloc (or any CUDA device pointer). Replaces the
 * "data pointer is a VulkanBuffer*" lookup of getDeviceFromPtr (src/api/hook.cpp:58-61). */
TVK_API int tvk_pointer_device(const void* ptr, int* dev);

/* Events on a device's compute stream. The reference's events are host clock stamps taken after a
 * flush (src/api/guard.cpp:44-62); these are recorded in stream order and timed on the device. */
TVK_API int tvk_event_create(void** event);
TVK_API int tvk_event_destroy(void* event);
TVK_API int tvk_event_record(int dev, void* event);
/* Work submitted to `dev`'s stream after this call runs after `event` (recorded on any device) has completed; the host does
 * not wait (the guard's block(), src/api/guard.cpp:60-75, whose streams are not real in the reference). */
TVK_API int tvk_event_wait(int dev, void* event);
TVK_API int tvk_event_synchronize(void* event);
TVK_API int tvk_event_query(void* event, int* done);
TVK_API int tvk_event_elapsed_ms(void* start, void* end, float* ms);

/* Step replay. The reference batches the operators of a step into one submission (its deferred op list and hazard
 * DAG, src/vulkan/shader.cpp:100-121, src/vulkan/dispatch.cpp:65-169); here the device's in-order stream is captured
 * into a CUDA graph and the whole step is replayed with one call. Between begin and end every launch of this library
 * on `dev` is recorded instead of run; calls that wait for the device (tvk_synchronize, tvk_memcpy_d2h, host-to-device
 * copies from pageable memory) fail while a capture is open. A replay reads and writes the buffers the captured step
 * used. Blocks tvk_malloc hands out while the capture runs join a pool owned by the graph: when they are freed (during
 * the capture or later) they are parked in that pool - reused inside the same capture only - and reach the shared
 * cache or the driver only with tvk_graph_destroy, so no later allocation is given memory that a replay writes into.
 * Inside a capture tvk_empty_cache is a no-op and an allocation the driver refuses fails with TVK_ERR_OOM at once (the
 * usual free-the-cache-and-retry step would wait for the device). Blocks that were allocated BEFORE the capture (the
 * model, the inputs) are the caller's to keep alive. tvk_graph_destroy waits for the device's stream first. */
TVK_API int tvk_graph_begin_capture(int dev);
TVK_API int tvk_graph_end_capture(int dev, void** graph);     /* instantiated, ready for tvk_graph_launch */
TVK_API int tvk_graph_launch(int dev, void* graph);
TVK_API int tvk_graph_destroy(void* graph);

/* Philox seed/offset bookkeeping of VulkanGeneratorImpl (src/vulkan/generator.cpp:82-168):
 * reserve() hands out one offset per launch. */
TVK_API int tvk_rng_set_seed(int dev, uint64_t seed);
TVK_API int tvk_rng_get_state(int dev, uint64_t* seed, uint64_t* offset);
TVK_API int tvk_rng_set_state(int dev, uint64_t seed, uint64_t offset);
TVK_API int tvk_rng_reserve(int dev, uint64_t count, uint64_t* seed, uint64_t* offset);
/* The same for a launch that may be recorded into a graph: outside a capture *device_state is NULL and (seed, offset) are
 * the reserved values; during tvk_graph_begin_capture .. tvk_graph_end_capture *device_state points at two words of device
 * memory (seed, base offset) that every tvk_graph_launch refreshes from the generator before the graph runs, and *offset
 * is relative to that base - so each replay draws new numbers and advances the generator by what the graph consumes. */
TVK_API int tvk_rng_reserve_state(int dev, uint64_t count, uint64_t* seed, uint64_t* offset, const uint64_t** device_state);
/* Random fills and dropout on a (seed, offset) pair reserved with tvk_rng_reserve (the reference's random family,
 * src/api/ops/random.cpp, and native_dropout_vulkan, src/api/ops/dropout.cpp:10-90). Philox4x32-10, four elements per
 * 128-bit block: a call over n elements consumes (n + 3) / 4 offsets. kind 0: uniform in [a, b); 1: normal(mean a,
 * std b); 2: Bernoulli(p = a) as 0 / 1 (dtype may be TVK_U8 for a mask). The streams are this library's own: the same
 * seed gives the same numbers here, not the reference's. tvk_dropout: out = keep ? in / keep_prob : 0, mask = keep.
 * device_state: NULL, or the pointer tvk_rng_reserve_state returned (the kernel then reads seed and base offset there). */
TVK_API int tvk_random_fill(int kind, int dtype, void* out, int64_t n, double a, double b, uint64_t seed, uint64_t offset,
                            const uint64_t* device_state, void* stream);
TVK_API int tvk_dropout(int dtype, void* out, uint8_t* mask, const void* in, int64_t n, double keep_prob, uint64_t seed,
                        uint64_t offset, const uint64_t* device_state, void* stream);

/* ------------------------------------------------------------------------- *
 * Dense contraction.
 * Replaces dispatch_matmul_coop_shader / dispatch_matmul_simd_shader
 * (src/api/ops/matmul.cpp:250-329, 373-582) and the matmul_coop / matmul_simd
 * shaders with their epilogue (src/shaders/ops/matmul_coop.slang:364-415).
 * ------------------------------------------------------------------------- */

typedef enum tvk_activation {
    TVK_ACT_NONE = 0,
    TVK_ACT_RELU = 1,
    TVK_ACT_GELU = 2  /* exact erf form, src/shaders/core/dtype.slang:736-737 */
} tvk_activation;

/* C[b] = act(alpha * A[b] @ B[b] + beta * bias[b]);  A is m x k, B is k x n, C is m x n.
 * Strides are in elements. A and B may have either stride equal to 1 (row- or
 * column-major, i.e. transposed views are consumed in place as the reference does,
 * src/api/ops/matmul.cpp:342-353). C rows are contiguous (c_cs == 1 implied).
 * bias may be NULL; its strides may be 0 for broadcast (matmul.cpp:49-53).
 * dtype is the type of A, B, C and bias: TVK_F16/TVK_BF16 accumulate in fp32
 * (matmul.cpp:92-95); TVK_F32 runs as a 3xTF32 split on the tensor cores. */
enum { TVK_AUX_NONE = 0, TVK_AUX_GELU_BACKWARD = 1, TVK_AUX_RELU_BACKWARD = 2 };

typedef struct tvk_gemm_desc {
    int32_t dtype;
    int32_t activation;
    int64_t batch, m, n, k;
    const void* a; int64_t a_rs, a_cs, a_bs;
    const void* b; int64_t b_rs, b_cs, b_bs;
    void* c;       int64_t c_rs, c_bs;
    const void* bias; int64_t bias_rs, bias_cs, bias_bs;
    float alpha, beta;
    int32_t force_path;  /* 0 = choose; 1 = tensor-core path or fail; 2 = CUDA-core path */
    int32_t c_f32;       /* != 0: C (and bias) are fp32 although A and B are fp16/bf16 (tensor-core path only) */
    /* Pushed copies (tensor-core path only; no counterpart in the reference, whose devices are independent,
     * src/vulkan/vulkan_context.cpp:626-631): the epilogue also stores every finished tile into peer_c[0..n_peer_c),
     * buffers with C's strides in OTHER devices' memory mapped into this process (tvk_ipc_open, or a pointer of a
     * peer-enabled device of this process). A batch-sharded bmm passes its slice of each peer's full output here, so
     * the all-gather rides on the epilogue stores over NVLink instead of following the GEMM. The kernel waits for
     * nothing; completion on the peers is the caller's (a stream-ordered barrier across the ranks). */
    int32_t n_peer_c;
    int32_t reserved_;
    void* peer_c[7];
    /* Epilogue fusion across the operator boundaries the reference's API exposes one by one (tensor-core path, fp16 /
     * bf16, no peer copies; other launches answer TVK_ERR_UNSUPPORTED and the caller issues the separate operators).
     * All NULL / 0 = plain behaviour.
     *   c2      second output with C's strides: C then receives alpha*A@B + beta*bias WITHOUT the activation (what
     *           backward needs) and c2 the activated value (what the next layer reads): addmm + gelu/relu
     *           (src/api/ops/matmul.cpp:670-683 keeps only one of the two) in one pass over the accumulator.
     *   aux     per-element operand of C's shape and dtype (row pitch aux_rs, batch pitch aux_bs, contiguous columns).
     *           aux_op TVK_AUX_GELU_BACKWARD: C = v * gelu'(aux) (erf form, src/shaders/core/dtype.slang:739-744), i.e.
     *           mm followed by gelu_backward with aux the saved pre-activation; TVK_AUX_RELU_BACKWARD: C = aux > 0 ? v : 0
     *           (threshold_backward). Applied after alpha and bias, before the activation. */
    void* c2;
    const void* aux;
    int64_t aux_rs, aux_bs;
    int32_t aux_op;
    int32_t reserved2_;
} tvk_gemm_desc;

/* Sharing a device buffer between the one-process-per-GPU ranks of a node (no counterpart in the reference).
 * tvk_ipc_export describes `ptr` (any address inside a device allocation made by this process, from tvk_malloc or
 * from another CUDA allocator that uses plain device allocations) as 72 opaque bytes; another process passes them
 * to tvk_ipc_open and receives an address in its own address space that refers to the same memory with peer
 * access enabled. tvk_ipc_close unmaps what tvk_ipc_open returned. The exporter must keep the allocation alive
 * until every importer has closed it. */
typedef struct tvk_ipc_handle {
    unsigned char reserved[64];
    uint64_t offset;
} tvk_ipc_handle;
TVK_API int tvk_ipc_export(const void* ptr, tvk_ipc_handle* handle);
TVK_API int tvk_ipc_open(const tvk_ipc_handle* handle, void** ptr);
TVK_API int tvk_ipc_close(void* ptr);

/* Scratch needed by tvk_gemm for this problem (0 for most fp16/bf16 problems). */
TVK_API int tvk_gemm_workspace_size(const tvk_gemm_desc* d, uint64_t* bytes);
TVK_API int tvk_gemm(const tvk_gemm_desc* d, void* workspace, uint64_t workspace_bytes, void* stream);
/* Which path tvk_gemm would take: 1 = tcgen05 tensor-core kernel, 2 = CUDA-core kernel. */
TVK_API int tvk_gemm_path(const tvk_gemm_desc* d, int* path);
/* How many K slices the tensor-core path would cut this product into (1 = a single launch). With more than one, the
 * slices' fp32 partials are summed by a finishing pass that applies bias, activation, c2 and aux - there the
 * fused forms cost no tensor-core epilogue time (the counterpart of the reference's split-K partials + at::sum,
 * src/api/ops/conv.cpp:1034-1060, and of its autotuner's split choice, src/vulkan/autotuner.cpp:123-178). */
TVK_API int tvk_gemm_splits(const tvk_gemm_desc* d, int* splits);
/* _scaled_mm: out = cast((A * scale_a) @ (B * scale_b) + bias), A [m, k] and B [k, n] float8 (e4m3fn or e5m2) with
 * element strides, scales fp32 in device memory: one value each (stride 0) or one per row of A and one per column of B
 * (stride 1). Replaces scaled_mm_out_vulkan (src/api/ops/matmul.cpp:706-747), which upcasts both operands to fp32, scales
 * them and multiplies in fp32; here the float8 values are widened exactly to fp16 and multiplied on the tensor cores with
 * fp32 accumulation, the scales applied to the accumulator. out is contiguous [m, n] of out_kind; bias ([n], fp32 / fp16
 * / bf16) may be NULL; scale_result (may be NULL) divides the result only for float8 outputs, as in the reference.
 * A float8 output is cast without saturation. The workspace must be 256-byte aligned. */
enum { TVK_F8_E4M3 = 0, TVK_F8_E5M2 = 1 };
enum { TVK_SCALED_OUT_F32 = 0, TVK_SCALED_OUT_F16 = 1, TVK_SCALED_OUT_BF16 = 2, TVK_SCALED_OUT_E4M3 = 3, TVK_SCALED_OUT_E5M2 = 4 };
typedef struct tvk_scaled_mm_desc {
    int32_t a_kind, b_kind, out_kind, bias_dtype;
    int64_t m, n, k;
    const void* a; int64_t a_rs, a_cs;
    const void* b; int64_t b_rs, b_cs;
    void* out;
    const float* scale_a; int64_t sa_stride;
    const float* scale_b; int64_t sb_stride;
    const void* bias;
    const float* scale_result;
} tvk_scaled_mm_desc;
TVK_API int tvk_scaled_mm_workspace_size(const tvk_scaled_mm_desc* d, uint64_t* bytes);
TVK_API int tvk_scaled_mm(const tvk_scaled_mm_desc* d, void* workspace, uint64_t workspace_bytes, void* stream);

/* Tuning hook of the tensor-core path, process-wide (the counterpart of pinning an entry of the reference's autotune
 * cache, src/vulkan/autotuner.cpp:123-178; used by sweeps and tests, not needed for normal use). 0 keeps the library's
 * choice. bn: tile width 32/64/128/256; mt: 128-row tiles per CTA block (1, 2); splits: K slices; group_m: tile rows
 * per raster group; debug: bit flags of timing probes (1: the epilogue stores nothing, 2: nothing is loaded or
 * multiplied, 4: staged tiles are not stored - results are then undefined). */
TVK_API int tvk_debug_gemm_tuning(int bn, int mt, int splits, int group_m, int debug);

/* ------------------------------------------------------------------------- *
 * Elementwise maps.
 * Replace unary_op_vulkan (src/api/ops/unary.cpp:76-135), dispatch_binary_shader
 * (src/api/ops/binary.cpp:60-131), dispatch_addc_shader (binary.cpp:711-771), the
 * compare/where/fill/cast/copy hosts and their shaders.
 * ------------------------------------------------------------------------- */

typedef enum tvk_unary_op {
    TVK_U_NEG = 0, TVK_U_EXP, TVK_U_LOG, TVK_U_SQRT, TVK_U_RSQRT, TVK_U_SIGMOID, TVK_U_RELU,
    TVK_U_GELU, TVK_U_TANH, TVK_U_ABS, TVK_U_SILU, TVK_U_RECIPROCAL, TVK_U_SQUARE,
    TVK_U_SIN, TVK_U_COS,
    TVK_U_GELU_TANH,          /* gelu(approximate='tanh'), src/shaders/core/dtype.slang:738 */
    /* the rest of the reference's unary family (src/api/ops/unary.cpp:137-260, one shader entry each) */
    TVK_U_FLOOR, TVK_U_CEIL, TVK_U_ROUND /* half to even */, TVK_U_TRUNC, TVK_U_SIGN,
    TVK_U_LOG2, TVK_U_LOG10, TVK_U_LOG1P, TVK_U_EXPM1, TVK_U_EXP2,
    TVK_U_TAN, TVK_U_SINH, TVK_U_COSH, TVK_U_ASIN, TVK_U_ACOS, TVK_U_ATAN, TVK_U_ERF, TVK_U_ERFC,
    TVK_U_HARDSIGMOID, TVK_U_HARDSWISH, TVK_U_MISH, TVK_U_LOGSIGMOID,
    TVK_U_ASINH, TVK_U_ACOSH, TVK_U_ATANH, TVK_U_ERFINV, TVK_U_LGAMMA, TVK_U_FRAC, TVK_U_SINC,
    TVK_U_COUNT_
} tvk_unary_op;

typedef enum tvk_binary_op {
    TVK_B_ADD = 0,            /* out = a + alpha*b                                          */
    TVK_B_SUB,                /* out = a - alpha*b                                          */
    TVK_B_MUL, TVK_B_DIV, TVK_B_MAXIMUM, TVK_B_MINIMUM, TVK_B_POW,
    TVK_B_GELU_BACKWARD,      /* a = grad, b = x (src/shaders/core/dtype.slang:739-751)     */
    TVK_B_THRESHOLD_BACKWARD, /* a = grad, b = x, alpha = threshold: x <= thr ? 0 : grad    */
    TVK_B_SILU_BACKWARD,      /* a = grad, b = x                                            */
    TVK_B_SIGMOID_BACKWARD,   /* a = grad, b = y                                            */
    TVK_B_TANH_BACKWARD,      /* a = grad, b = y                                            */
    TVK_B_GELU_TANH_BACKWARD, /* a = grad, b = x (src/shaders/core/dtype.slang:745-751)     */
    TVK_B_ADD_RELU,           /* out = relu(a + alpha*b): _add_relu, which the reference runs as add then relu
                                 (src/api/ops/binary.cpp:655-673), in one pass; NaN propagates as in relu */
    TVK_B_FMOD,               /* C fmod: the result has the sign of a                        */
    TVK_B_REMAINDER,          /* Python %: the result has the sign of b                      */
    TVK_B_ATAN2,
    TVK_B_FLOOR_DIVIDE,       /* floor(a / b) with ATen's correction for the rounding of a / b */
    /* one tensor and two scalars (b == NULL: b_scalar and alpha are the parameters) */
    TVK_B_CLAMP,              /* min(max(a, alpha), b_scalar), NaN stays NaN (also hardtanh) */
    TVK_B_LEAKY_RELU,         /* a > 0 ? a : a * b_scalar                                    */
    TVK_B_ELU,                /* a > 0 ? a : alpha * (exp(a) - 1)                            */
    TVK_B_SOFTPLUS,           /* beta = alpha, threshold = b_scalar                          */
    /* gradients: a = grad, b = x */
    TVK_B_LEAKY_RELU_BACKWARD,   /* alpha = negative slope                                   */
    TVK_B_ELU_BACKWARD,          /* alpha as in the forward, b = the input                   */
    TVK_B_HARDSWISH_BACKWARD, TVK_B_HARDSIGMOID_BACKWARD, TVK_B_MISH_BACKWARD, TVK_B_LOGSIGMOID_BACKWARD,
    TVK_B_SOFTPLUS_BACKWARD,     /* beta = alpha, threshold 20                               */
    TVK_B_HYPOT, TVK_B_COPYSIGN, TVK_B_LOGADDEXP, TVK_B_LOGADDEXP2,
    TVK_B_FMAX, TVK_B_FMIN,      /* maximum / minimum that ignore a NaN operand              */
    TVK_B_HEAVISIDE,             /* a < 0 ? 0 : a > 0 ? 1 : b                                */
    TVK_B_COUNT_
} tvk_binary_op;

typedef enum tvk_compare_op {
    TVK_C_EQ = 0, TVK_C_NE, TVK_C_LT, TVK_C_LE, TVK_C_GT, TVK_C_GE, TVK_C_COUNT_
} tvk_compare_op;

typedef enum tvk_ternary_op {
    TVK_T_ADDCMUL = 0,  /* out = a + value * b * c  (src/shaders/ops/addc.slang:62-68)      */
    TVK_T_ADDCDIV,      /* out = a + value * b / c                                          */
    TVK_T_LERP,         /* out = a + value * (b - a), scalar weight; c unused              */
    TVK_T_WHERE,        /* out = cond(c: u8) ? a : b                                        */
    TVK_T_COUNT_
} tvk_ternary_op;

/* Iteration space of a strided/broadcast elementwise call: `ndim` sizes and, per operand,
 * element strides (0 = broadcast). Operand 0 is the output. Mirrors the TensorIterator →
 * metadata packing of src/api/ops/helpers.h:198-234. */
typedef struct tvk_iter {
    int32_t ndim;
    int32_t noperands;
    int64_t sizes[TVK_MAX_DIMS];
    int64_t strides[4][TVK_MAX_DIMS];
} tvk_iter;

/* Contiguous fast paths: n elements, 128-bit accesses. A NULL `b` (binary) means the scalar
 * operand `b_scalar` is used instead (the scalar-operand variants of binary.cpp). */
TVK_API int tvk_unary(int op, int dtype, void* out, const void* in, int64_t n, void* stream);
TVK_API int tvk_binary(int op, int dtype, void* out, const void* a, const void* b, double b_scalar,
                       double alpha, int64_t n, void* stream);
TVK_API int tvk_compare(int op, int dtype, uint8_t* out, const void* a, const void* b, double b_scalar,
                        int64_t n, void* stream);
/* Logical and / or / xor / not on boolean tensors (one byte per element, any non-zero byte is true, results are 0 or 1):
 * logical_and/or/xor/not of src/api/ops/compare.cpp (dispatch_compare_shader), contiguous operands. b is ignored for NOT. */
typedef enum tvk_logical_op { TVK_L_AND = 0, TVK_L_OR, TVK_L_XOR, TVK_L_NOT, TVK_L_COUNT_ } tvk_logical_op;
TVK_API int tvk_logical(int op, uint8_t* out, const uint8_t* a, const uint8_t* b, int64_t n, void* stream);
TVK_API int tvk_ternary(int op, int dtype, void* out, const void* a, const void* b, const void* c,
                        double value, int64_t n, void* stream);
/* Strided/broadcast variants over a tvk_iter. */
TVK_API int tvk_unary_strided(int op, int dtype, void* out, const void* in, const tvk_iter* it, void* stream);
TVK_API int tvk_binary_strided(int op, int dtype, void* out, const void* a, const void* b, double alpha,
                               const tvk_iter* it, void* stream);
TVK_API int tvk_compare_strided(int op, int dtype, uint8_t* out, const void* a, const void* b,
                                const tvk_iter* it, void* stream);
TVK_API int tvk_ternary_strided(int op, int dtype, void* out, const void* a, const void* b, const void* c,
                                double value, const tvk_iter* it, void* stream);
/* fill (src/shaders/ops/fill.slang), dtype cast (src/api/tensor/cast.cpp:8-55; contiguous n
 * elements), strided copy with optional cast (src/api/tensor/transfer.cpp:16-56). */
TVK_API int tvk_fill(int dtype, void* out, double value, int64_t n, void* stream);
TVK_API int tvk_cast(int dst_dtype, void* dst, int src_dtype, const void* src, int64_t n, void* stream);
TVK_API int tvk_copy_strided(int dst_dtype, void* dst, int src_dtype, const void* src, const tvk_iter* it,
                             void* stream);

/* ------------------------------------------------------------------------- *
 * Reductions.
 * Replace dispatch_reduce_shader / reduce_dims_vulkan (src/api/ops/reduce.cpp:26-121,
 * 207-284) and argreduce (reduce.cpp:424-502, src/shaders/ops/arg_reduce.slang:26-66).
 * The input is viewed as [outer, reduce, inner] contiguous; the output is [outer, inner].
 * ------------------------------------------------------------------------- */

typedef enum tvk_reduce_op {
    TVK_R_SUM = 0, TVK_R_MEAN, TVK_R_AMAX, TVK_R_AMIN, TVK_R_COUNT_
} tvk_reduce_op;

/* Scratch for tvk_reduce / tvk_argreduce on this shape (partials of multi-block lines). */
TVK_API int tvk_reduce_workspace_size(int64_t outer, int64_t reduce, int64_t inner, uint64_t* bytes);
/* in_dtype f32/f16/bf16; accumulation in fp32 (reduce.cpp:266-274); out_dtype may differ
 * from in_dtype (e.g. fp16 in, fp32 out). */
TVK_API int tvk_reduce(int op, int in_dtype, int out_dtype, void* out, const void* in, int64_t outer,
                       int64_t reduce, int64_t inner, void* workspace, uint64_t workspace_bytes,
                       void* stream);
/* tvk_reduce for callers that cannot allocate (no counterpart in the reference). A host that
 * may not call cudaMalloc when it needs the reduction (it runs inside a pool that owns the device,
 * or its application forbids driver allocations after start-up) passes inputs and outputs only:
 * the per-CTA partials live in a fixed 128 KiB array inside the library image, held on every GPU
 * that loads the library until the process exits. Shapes whose partials exceed it (more than
 * 8192 partials; see tvk_reduce_workspace_size) return TVK_ERR_INVALID. All calls share the
 * array, so calls that overlap on the GPU race; calls on one stream are ordered and safe. The
 * first call on each device resolves the array's device address and should be made outside
 * stream capture. It never calls cudaMalloc/cudaFree or an allocating library routine. */
TVK_API int tvk_reduce_noalloc(int op, int in_dtype, int out_dtype, void* out, const void* in, int64_t outer,
                               int64_t reduce, int64_t inner, void* stream);
/* Index (int64) of the first maximal / minimal element of every line; NaN counts as the
 * extreme and the first NaN wins (arg_reduce.slang:49-65). */
TVK_API int tvk_argreduce(int is_max, int dtype, int64_t* out, const void* in, int64_t outer,
                          int64_t reduce, int64_t inner, void* workspace, uint64_t workspace_bytes,
                          void* stream);

/* ------------------------------------------------------------------------- *
 * Row-wise kernels: softmax family, losses, norms, embedding.
 * ------------------------------------------------------------------------- */

/* softmax / log_softmax over the last dimension of a contiguous [rows, cols] view, fp32 math,
 * one rounding (src/api/decompositions.cpp:506-571). in/out dtypes may differ (half in,
 * float out is the `half_to_float` flag). */
TVK_API int tvk_softmax_forward(int is_log, int in_dtype, int out_dtype, void* out, const void* in,
                                int64_t rows, int64_t cols, void* stream);
/* grad_in = softmax: y*(g - sum(g*y));  log_softmax: g - exp(y)*sum(g). */
TVK_API int tvk_softmax_backward(int is_log, int dtype, void* grad_in, const void* grad_out,
                                 const void* out, int64_t rows, int64_t cols, void* stream);

/* nll_loss forward/backward (src/api/ops/nllloss.cpp:79-174, src/shaders/ops/nllloss.slang:20-65).
 * logp is [n, c]; target int64 [n]; weight may be NULL; reduction: 0 none, 1 mean, 2 sum.
 * Targets equal to ignore_index or outside [0, c) contribute 0. `out` has n elements for
 * reduction none, else 1; total_weight has 1 element (both of `dtype`). */
TVK_API int tvk_nll_loss_forward(int dtype, void* out, void* total_weight, const void* logp,
                                 const int64_t* target, const void* weight, int64_t n, int64_t c,
                                 int reduction, int64_t ignore_index, void* stream);
/* grad_in [n, c] is fully written (zeros elsewhere). grad_out has n elements (none) or 1. */
TVK_API int tvk_nll_loss_backward(int dtype, void* grad_in, const void* grad_out, const int64_t* target,
                                  const void* weight, const void* total_weight, int64_t n, int64_t c,
                                  int reduction, int64_t ignore_index, void* stream);

/* LayerNorm (layer_norm_shader / layer_norm_backward_shader, src/api/ops/norm.cpp:264-325; rowForward, rowBackwardInput,
 * rowBackwardParams of src/shaders/ops/norm.slang:193-317). x viewed as [rows, cols] contiguous with cols the product of
 * normalized_shape. y = (x - mean) * rstd * w + b; mean and rstd (biased variance, two-pass) saved as fp32 [rows].
 * weight / bias may be NULL. */
TVK_API int tvk_layernorm_forward(int dtype, void* y, float* mean, float* rstd, const void* x, const void* weight,
                                  const void* bias, int64_t rows, int64_t cols, double eps, void* stream);
/* Any of grad_x, grad_w, grad_b may be NULL. grad_w / grad_b (cols, `dtype`) need fp32 scratch of
 * tvk_layernorm_backward_workspace_size bytes. cols <= 8192. */
TVK_API int tvk_layernorm_backward_workspace_size(int64_t rows, int64_t cols, uint64_t* bytes);
TVK_API int tvk_layernorm_backward(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y, const void* x,
                                   const void* weight, const float* mean, const float* rstd, int64_t rows, int64_t cols,
                                   void* workspace, uint64_t workspace_bytes, void* stream);
/* GroupNorm over contiguous [n, channels, hw] (native_group_norm, src/api/ops/norm.cpp:264-325 row mode with per-channel
 * affine): mean / rstd fp32 [n, groups]. */
TVK_API int tvk_groupnorm_forward(int dtype, void* y, float* mean, float* rstd, const void* x, const void* weight,
                                  const void* bias, int64_t n, int64_t channels, int64_t hw, int64_t groups, double eps,
                                  void* stream);
TVK_API int tvk_groupnorm_backward(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y, const void* x,
                                   const void* weight, const float* mean, const float* rstd, int64_t n, int64_t channels,
                                   int64_t hw, int64_t groups, void* stream);

/* Cross-entropy of [n, c] logits with class-index targets in one pass each way: what the reference runs as log_softmax
 * (src/api/decompositions.cpp:506-571) followed by nll_loss (src/api/ops/nllloss.cpp:79-174), without the [n, c] table
 * of log-probabilities in between. Same conventions as tvk_nll_loss_*: reduction 0 none (loss has n elements), 1 mean
 * (sum of w[t] * loss / sum of w[t]), 2 sum; targets equal to ignore_index or outside [0, c) contribute nothing.
 * lse (fp32 [n], may be NULL) receives the row log-sum-exp, which the backward pass needs. total_weight (may be NULL)
 * as nll_loss_forward's second result. Reductions other than none need tvk_cross_entropy_workspace_size bytes. */
TVK_API int tvk_cross_entropy_workspace_size(int64_t n, uint64_t* bytes);
TVK_API int tvk_cross_entropy_forward(int dtype, void* loss, void* total_weight, float* lse, const void* logits,
                                      const int64_t* target, const void* weight, int64_t n, int64_t c, int reduction,
                                      int64_t ignore_index, void* workspace, uint64_t workspace_bytes, void* stream);
/* grad_logits[i, j] = (softmax(logits_i)[j] - [j == target_i]) * w[target_i] * grad_out (/ total_weight for the mean). */
TVK_API int tvk_cross_entropy_backward(int dtype, void* grad_logits, const void* grad_out, const void* logits,
                                       const float* lse, const int64_t* target, const void* weight,
                                       const void* total_weight, int64_t n, int64_t c, int reduction,
                                       int64_t ignore_index, void* stream);

/* Inclusive scan along the middle axis of a contiguous [outer, n, inner] view (cumscan, src/api/ops/scan.cpp:35-102;
 * src/shaders/ops/scan.slang): cumsum, cumprod, logcumsumexp. Floating types accumulate in fp32 and round every
 * output; TVK_I64 scans in int64 (sum and product). */
enum { TVK_SCAN_SUM = 0, TVK_SCAN_PROD = 1, TVK_SCAN_LOGADDEXP = 2 };
TVK_API int tvk_scan(int op, int dtype, void* out, const void* in, int64_t outer, int64_t n, int64_t inner, void* stream);

/* RMSNorm (src/api/ops/norm.cpp:169-260; src/shaders/ops/norm.slang:193-317).
 * y = x * rstd * w, rstd = rsqrt(mean(x^2) + eps) saved as fp32 [rows]. weight may be NULL. */
TVK_API int tvk_rmsnorm_forward(int dtype, void* y, float* rstd, const void* x, const void* weight,
                                int64_t rows, int64_t cols, double eps, void* stream);
/* grad_x always; grad_w (cols, `dtype`) if non-NULL, using fp32 scratch of
 * tvk_rmsnorm_backward_workspace_size bytes. */
TVK_API int tvk_rmsnorm_backward_workspace_size(int64_t rows, int64_t cols, uint64_t* bytes);
TVK_API int tvk_rmsnorm_backward(int dtype, void* grad_x, void* grad_w, const void* grad_y, const void* x,
                                 const void* weight, const float* rstd, int64_t rows, int64_t cols,
                                 void* workspace, uint64_t workspace_bytes, void* stream);

/* Training-mode batch norm over NCHW (src/api/ops/norm.cpp:327-428, norm.slang:72-191).
 * x,y: [n, c, hw]; per-channel stats in fp32. save_mean / save_invstd are outputs (fp32 [c]).
 * running_mean/var (of `stat_dtype`, may be NULL) are updated with momentum using the unbiased
 * variance (norm.slang:99-113). */
TVK_API int tvk_batchnorm_workspace_size(int64_t n, int64_t c, int64_t hw, uint64_t* bytes);
TVK_API int tvk_batchnorm_forward(int dtype, void* y, float* save_mean, float* save_invstd, const void* x,
                                  const void* weight, const void* bias, int stat_dtype, void* running_mean,
                                  void* running_var, int64_t n, int64_t c, int64_t hw, double momentum,
                                  double eps, void* workspace, uint64_t workspace_bytes, void* stream);
/* grad_x, grad_w, grad_b (any may be NULL). */
TVK_API int tvk_batchnorm_backward(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y,
                                   const void* x, const void* weight, const float* save_mean,
                                   const float* save_invstd, int64_t n, int64_t c, int64_t hw,
                                   void* workspace, uint64_t workspace_bytes, void* stream);
/* The same for channels-last data: x, y, grad_x, grad_y are [rows = n*hw, c] with the channel contiguous (a
 * tensor of torch.channels_last memory format, the layout conv2d also takes; the reference keeps the input's
 * memory format, src/api/ops/conv.cpp:1080-1086). c must be a multiple of 16 bytes' worth of elements and the
 * tensors 16-byte aligned, else TVK_ERR_UNSUPPORTED (callers fall back to the NCHW entry points on a copy). */
/* Evaluation mode (batch_norm with training == false, src/api/ops/norm.cpp:177): y = (x - running_mean) *
 * rsqrt(running_var + eps) * weight + bias, one pass. x and y are [n, c, hw] (channels_last == 0) or [n*hw, c]
 * (channels_last != 0); the statistics are stat_dtype (f32/f16/bf16), weight and bias (either may be NULL) are dtype. */
TVK_API int tvk_batchnorm_inference(int dtype, void* y, const void* x, const void* weight, const void* bias, int stat_dtype,
                                    const void* running_mean, const void* running_var, int64_t n, int64_t c, int64_t hw,
                                    int channels_last, double eps, void* stream);
TVK_API int tvk_batchnorm_cl_workspace_size(int64_t rows, int64_t c, uint64_t* bytes);
TVK_API int tvk_batchnorm_forward_cl(int dtype, void* y, float* save_mean, float* save_invstd, const void* x,
                                     const void* weight, const void* bias, int stat_dtype, void* running_mean,
                                     void* running_var, int64_t rows, int64_t c, double momentum, double eps,
                                     void* workspace, uint64_t workspace_bytes, void* stream);
TVK_API int tvk_batchnorm_backward_cl(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y,
                                      const void* x, const void* weight, const float* save_mean,
                                      const float* save_invstd, int64_t rows, int64_t c, void* workspace,
                                      uint64_t workspace_bytes, void* stream);

/* Embedding forward = row gather (src/api/ops/indexing.cpp:299-314): out[i, :] = table[idx[i], :].
 * Indices outside [0, num_rows) write zeros and raise the device status word. */
TVK_API int tvk_embedding_forward(int dtype, void* out, const void* table, const int64_t* idx,
                                  int64_t num_idx, int64_t num_rows, int64_t dim, void* stream);
/* Deterministic dense backward (src/shaders/ops/embedding_backward.slang:36-56): grad_table[r, :]
 * = sum over i with idx[i] == r (and r != padding_idx) of grad[i, :], summed in fp32 in
 * increasing i. */
TVK_API int tvk_embedding_backward(int dtype, void* grad_table, const void* grad, const int64_t* idx,
                                   int64_t num_idx, int64_t num_rows, int64_t dim, int64_t padding_idx,
                                   void* stream);

/* Scaled dot-product attention with grouped-query heads (sdpa_forward_vulkan / sdpa_backward_vulkan,
 * src/api/ops/attention.cpp:395-480, 641-749; src/shaders/ops/attention_coop.slang). fp16 / bf16.
 * q, out, dq, dout: contiguous [B, Hq, L, D]; k, v, dk, dv: contiguous [B, Hk, S, D]; Hq % Hk == 0 and
 * query head h reads key/value head h / (Hq/Hk). lse: fp32 [B, Hq, L]. causal != 0 masks key j of
 * query l when j > l (top-left aligned when L != S, as src/api/ops/attention.cpp:107-112 and ATen's is_causal do).
 * A row with no visible key (lse = +inf) gives out = 0 and zero gradients.
 * D and S must be multiples of 8. */
TVK_API int tvk_attention_workspace_size(int dtype, int64_t B, int64_t Hq, int64_t Hk, int64_t L, int64_t S,
                                         int64_t D, int backward, uint64_t* bytes);
TVK_API int tvk_attention_forward(int dtype, void* out, float* lse, const void* q, const void* k, const void* v,
                                  int64_t B, int64_t Hq, int64_t Hk, int64_t L, int64_t S, int64_t D, double scale,
                                  int causal, void* workspace, uint64_t workspace_bytes, void* stream);
TVK_API int tvk_attention_backward(int dtype, void* dq, void* dk, void* dv, const void* dout, const void* q,
                                   const void* k, const void* v, const void* out, const float* lse, int64_t B,
                                   int64_t Hq, int64_t Hk, int64_t L, int64_t S, int64_t D, double scale, int causal,
                                   void* workspace, uint64_t workspace_bytes, void* stream);

/* 2-D convolution, its input gradient and its weight gradient (convolution_vulkan and
 * convolution_backward_vulkan, src/api/ops/conv.cpp:1088-1172; dispatch_conv_shader conv.cpp:661-685;
 * the three modes FORWARD / GRAD_INPUT / GRAD_WEIGHT of conv.cpp:241-245). fp16 / bf16 with fp32
 * accumulation, and fp32. x, dx: contiguous NCHW [n, cin, h, w]; w, dw: contiguous OIHW [cout, cin, kh, kw];
 * y, dy: contiguous [n, cout, ho, wo] with ho = (h + 2*pad_h - dilation_h*(kh - 1) - 1) / stride_h + 1 (likewise wo).
 * fp16 / bf16 with stride_h == stride_w in {1, 2}, dilation 1 and kh*kw <= 64 run on the implicit-GEMM tensor-core
 * kernels; fp32 and every other stride, dilation and filter size run as unfold + GEMM + fold (the reference's own
 * im2col route, conv.cpp:200-216). groups must be 1 (see the depthwise entry points below); other dtypes
 * return TVK_ERR_UNSUPPORTED with a "[NOT IMPLEMENTED]" message. The bias and its gradient are
 * a broadcast add and a reduction (tvk_binary_strided, tvk_reduce) as in conv.cpp:1159-1170.
 * mode: 0 forward, 1 input gradient, 2 weight gradient, 3 both gradients (tvk_conv2d_backward); the workspace must
 * be 256-byte aligned. */
typedef struct tvk_conv2d_desc {
    int dtype;
    int64_t n, cin, h, w;
    int64_t cout, kh, kw;
    int64_t stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w, groups;
    /* Memory layout of the tensors, a sum of TVK_CONV_*_CHANNELS_LAST: 0 = NCHW / OIHW as above. A channels-last
     * tensor has the same logical shape stored as [n, h, w, c] (torch.channels_last; the reference's output format
     * follows its inputs, conv.cpp:1080-1086, 1112). Channels-last activations whose channel count is a multiple
     * of 8 are read and written in place by the kernels (no staging copy); this is the fast layout. */
    int64_t layout;
} tvk_conv2d_desc;
#define TVK_CONV_X_CHANNELS_LAST 1 /* x and dx */
#define TVK_CONV_Y_CHANNELS_LAST 2 /* y and dy */
#define TVK_CONV_W_CHANNELS_LAST 4 /* w and dw */
TVK_API int tvk_conv2d_workspace_size(const tvk_conv2d_desc* desc, int mode, uint64_t* bytes);
TVK_API int tvk_conv2d_forward(const tvk_conv2d_desc* desc, void* y, const void* x, const void* w, void* workspace,
                               uint64_t workspace_bytes, void* stream);
TVK_API int tvk_conv2d_backward_input(const tvk_conv2d_desc* desc, void* dx, const void* dy, const void* w,
                                      void* workspace, uint64_t workspace_bytes, void* stream);
TVK_API int tvk_conv2d_backward_weight(const tvk_conv2d_desc* desc, void* dw, const void* dy, const void* x,
                                       void* workspace, uint64_t workspace_bytes, void* stream);
/* Both gradients of one convolution in one call, as the reference's convolution_backward_vulkan computes them
 * (src/api/ops/conv.cpp:1126-1172): an NCHW dy is brought into the kernels' channels-last layout once for the two
 * products instead of once in each. dx or dw may be null (that gradient is skipped). Workspace: mode 3 of
 * tvk_conv2d_workspace_size. The results are bit-identical to the two separate calls. */
TVK_API int tvk_conv2d_backward(const tvk_conv2d_desc* desc, void* dx, void* dw, const void* dy, const void* x, const void* w,
                                void* workspace, uint64_t workspace_bytes, void* stream);

/* 2-D max and average pooling on NCHW planes (src/api/ops/pool.cpp: max_pool2d_with_indices, avg_pool2d and their
 * backward entries). planes = n * c; x, dx: [planes, h, w]; y, dy, indices: [planes, ho, wo], ho / wo given by the caller
 * (floor or ceil mode). Max pooling: a NaN in the window wins, ties keep the first element, indices[...] = h * w_in + w
 * inside the plane; average pooling: the divisor is divisor_override when > 0, else the window's size clipped to the
 * padded plane (count_include_pad != 0) or to the plane. The backward calls are gathers: deterministic, no atomics. */
typedef struct tvk_pool2d_desc {
    int dtype;
    int64_t planes, h, w, ho, wo;
    int64_t kh, kw, stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w;
    int32_t count_include_pad;
    int64_t divisor_override;
} tvk_pool2d_desc;
TVK_API int tvk_max_pool2d_forward(const tvk_pool2d_desc* desc, void* y, int64_t* indices, const void* x, void* stream);
TVK_API int tvk_max_pool2d_backward(const tvk_pool2d_desc* desc, void* dx, const void* dy, const int64_t* indices, void* stream);
TVK_API int tvk_avg_pool2d_forward(const tvk_pool2d_desc* desc, void* y, const void* x, void* stream);
TVK_API int tvk_avg_pool2d_backward(const tvk_pool2d_desc* desc, void* dx, const void* dy, void* stream);

/* Depthwise 2-D convolution: groups == cin, cout a multiple of cin (one input channel per group). The reference sends
 * these through the same grouped convolution as everything else (convolution_vulkan with groups > 1,
 * src/api/ops/conv.cpp:1088-1117; the depthwise / slow aliases conv.cpp:218-230). Direct kernels, fp32 / fp16 / bf16 with
 * fp32 accumulation, any stride, padding and dilation, NCHW tensors (layout must be 0): w and dw are [cout, 1, kh, kw].
 * The weight gradient supports filters of up to 49 taps and sums in a fixed order. */
TVK_API int tvk_depthwise_conv2d_forward(const tvk_conv2d_desc* desc, void* y, const void* x, const void* w, void* stream);
TVK_API int tvk_depthwise_conv2d_backward_input(const tvk_conv2d_desc* desc, void* dx, const void* dy, const void* w, void* stream);
TVK_API int tvk_depthwise_conv2d_backward_weight(const tvk_conv2d_desc* desc, void* dw, const void* dy, const void* x, void* stream);

/* Stable sort of every line of a contiguous [lines, n] view and top-k as "sort then take k"
 * (src/api/ops/sort.cpp:19-140): order by value (descending if `descending`), NaN largest,
 * ties by ascending original position (src/shaders/ops/sort.slang:24-49). values_out is
 * [lines, k], indices_out int64 [lines, k]; k == n gives the full sort. */
TVK_API int tvk_sort_workspace_size(int dtype, int64_t lines, int64_t n, uint64_t* bytes);
TVK_API int tvk_topk(int dtype, void* values_out, int64_t* indices_out, const void* in, int64_t lines,
                     int64_t n, int64_t k, int descending, void* workspace, uint64_t workspace_bytes,
                     void* stream);

/* ------------------------------------------------------------------------- *
 * Optimizer steps (src/api/ops/optim.cpp:46-126, 172-206), one fused pass each.
 * ------------------------------------------------------------------------- */

/* Adam/AdamW on n contiguous elements. Low-precision parameters compute in fp32 (optim.cpp:41-44).
 * step is the 1-based step count after increment; bias corrections are formed on the host in
 * double as the reference does. decoupled != 0 = AdamW (p *= 1 - lr*wd), else L2 (g += wd*p). */
TVK_API int tvk_adam_step(int dtype, void* param, const void* grad, void* exp_avg, void* exp_avg_sq,
                          int64_t n, double lr, double beta1, double beta2, double eps,
                          double weight_decay, int64_t step, int decoupled, int maximize, void* stream);
/* SGD with momentum (optim.cpp:200-204): g += wd*p; buf = first ? g : mu*buf + (1-dampening)*g;
 * g = nesterov ? g + mu*buf : buf; p -= lr*g. momentum_buf may be NULL when momentum == 0. */
TVK_API int tvk_sgd_step(int dtype, void* param, const void* grad, void* momentum_buf, int64_t n,
                         double lr, double momentum, double dampening, double weight_decay,
                         int nesterov, int maximize, int first_step, void* stream);

/* The same steps, and the in-place list updates of torch's foreach optimizers, over a LIST of tensors in
 * one launch per 24 tensors (the reference loops over the list with one dispatch chain per tensor:
 * fused_adam / fused_sgd optim.cpp:88-126, 172-206; foreach slow path binary.cpp:1039-1061). `items` is a
 * host array; every tensor of an item is dense with `numel` elements of `dtype`.
 *   adam:  ptr = {param, grad, exp_avg, exp_avg_sq}; step = device pointer to the 1-based step count held
 *          as fp32 (torch keeps it on the device for fused optimizers), or NULL to use host_step.
 *   sgd:   ptr = {param, grad, momentum_buf (unused when momentum == 0)}.
 *   axpby: ptr[0] = a (updated in place), ptr[1] = b when has_b:  a = scale_a*a + scale_b*b + add. */
typedef struct tvk_multi_item {
    void* ptr[4];
    int64_t numel;
    const float* step;
} tvk_multi_item;
TVK_API int tvk_adam_step_multi(int dtype, const tvk_multi_item* items, int count, double lr, double beta1,
                                double beta2, double eps, double weight_decay, int64_t host_step, int decoupled,
                                int maximize, void* stream);
TVK_API int tvk_sgd_step_multi(int dtype, const tvk_multi_item* items, int count, double lr, double momentum,
                               double dampening, double weight_decay, int nesterov, int maximize, int first_step,
                               void* stream);
TVK_API int tvk_foreach_axpby(int dtype, const tvk_multi_item* items, int count, double scale_a, double scale_b,
                              double add, int has_b, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TVK_H_ */
