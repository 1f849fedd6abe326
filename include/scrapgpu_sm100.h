/*
 * scrapgpu_sm100.h -- C ABI of libscrapgpu_sm100.so, the B200 (sm_100a) compute library underneath the
 * `cuda_sm100` backend of ScrapGpuLibrary.
 *
 * Plain pointers and sizes only.  Every function returns a scrapgpu_status value
 * (0 OK, 1 UNSUPPORTED, 2 INVALID_ARGUMENT, 3 OUT_OF_MEMORY, 4 BACKEND_ERROR; the reference's
 * include/scrapgpu/status.h:10-17) and leaves a message for sm100_last_error() on failure.
 * Tensor conventions are the reference's (ggml): W = [K, N] is N weight rows of K elements,
 * x = [K, M] is M activation columns, y = [N, M]; y[n,m] = sum_k W[k,n] x[k,m].
 * dtype codes are scrapgpu_dtype (include/scrapgpu/tensor.h:10-22): F32 0, F16 1, I32 2, Q4_0 16,
 * Q8_0 17, Q4_K 32, Q6_K 33.  layout codes are scrapgpu_layout (tensor.h:24-27): 0 = natural GGUF
 * blocks, 1 = backend-packed (the B200 plane layout produced by sm100_pack).
 *
 * Each entry names the reference interface it stands in for (file:line relative to the reference
 * project).  There is no CPU fallback anywhere in this library: without a CUDA device the compute
 * entry points fail with BACKEND_ERROR.
 */
#ifndef SCRAPGPU_SM100_H
#define SCRAPGPU_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SM100_API __attribute__((visibility("default")))

typedef void * sm100_stream_t; /* a cudaStream_t */
typedef void * sm100_event_t;  /* a cudaEvent_t */
typedef void * sm100_graph_t;  /* a cudaGraphExec_t */

/* A tensor as the backend vtable sees it (scrapgpu_tensor_desc, include/scrapgpu/tensor.h:29-37, with the
 * buffer already resolved to a device address): extents ne[4] (ne[0] contiguous-most) and byte strides nb[4]. */
typedef struct sm100_view {
    void * data;
    int64_t ne[4];
    int64_t nb[4];
} sm100_view;

/* ---- errors (src/core/status.cpp:6-37: thread-local last error) ---- */
SM100_API const char * sm100_last_error(void);

/* ---- devices, memory, streams: what a backend's device / buffer / stream vtable slots need
 *      (include/scrapgpu/backend.h:33-44; CPU counterparts src/backends/cpu/api.cpp:1040-1300) ---- */
SM100_API int sm100_device_count(void);
SM100_API int sm100_device_info(int device, char * name, size_t name_size, uint64_t * total_memory,
                                uint32_t * sm_count, uint32_t * cc_major, uint32_t * cc_minor,
                                uint64_t * shared_per_block);
SM100_API int sm100_set_device(int device);
SM100_API int sm100_malloc(int device, size_t size, void ** out);           /* buffer_alloc (256 B aligned) */
SM100_API int sm100_free(int device, void * ptr);                            /* buffer_free */
SM100_API int sm100_host_alloc(size_t size, void ** out);                    /* pinned staging memory */
SM100_API int sm100_host_free(void * ptr);
SM100_API int sm100_stream_create(int device, sm100_stream_t * out);         /* stream_create */
SM100_API int sm100_stream_destroy(int device, sm100_stream_t stream);       /* stream_free */
SM100_API int sm100_stream_sync(sm100_stream_t stream);                      /* stream_sync */
SM100_API int sm100_memcpy_h2d(sm100_stream_t s, void * dst, const void * src, size_t n, int blocking); /* buffer_write */
SM100_API int sm100_memcpy_d2h(sm100_stream_t s, void * dst, const void * src, size_t n, int blocking); /* buffer_read */
SM100_API int sm100_memcpy_d2d(sm100_stream_t s, void * dst, const void * src, size_t n, int blocking); /* buffer_copy (memmove semantics) */
SM100_API int sm100_memset(sm100_stream_t s, void * dst, int byte, size_t n, int blocking);            /* buffer_fill */
/* cross-device copy for scrapgpu_tensor_copy between two cuda_sm100 devices (src/core/transport.cpp:53-146):
 * ordered after the work on src_stream and before later work on dst_stream, no host bounce */
SM100_API int sm100_memcpy_peer(sm100_stream_t dst_stream, int dst_device, void * dst, sm100_stream_t src_stream,
                                int src_device, const void * src, size_t n);

/* lets kernels and copies running on `device` address memory allocated on `peer` (both in this process); UNSUPPORTED
 * when the two GPUs have no peer path.  Needed once per ordered pair before sm100_allreduce_* is used with areas that
 * live in the same process (ranks in separate processes map each other's areas with sm100_ipc_open instead). */
SM100_API int sm100_peer_access(int device, int peer);

/* ---- tensor-parallel exchange over peer-mapped memory (one process per GPU, or one process driving several) ----
 * The reference moves tensors between devices through a host bounce (src/core/transport.cpp:53-146) and has no
 * collective; the tensor-parallel decode needs an all-reduce of the hidden vector after the row-parallel projections.
 * Each rank allocates one area of sm100_allreduce_area_bytes() with sm100_malloc, zero-fills it, exports it
 * (sm100_ipc_export), and opens the other ranks' handles (sm100_ipc_open); `areas` lists all ranks' areas as seen from
 * this process (entry `rank` = the local pointer).  sm100_allreduce_sum is one single-CTA kernel: every value goes to every
 * peer as one 8-byte store carrying the call number as its tag (no fence, no flag), then the slots are added in rank order
 * (same bits on every rank) with a bounded wait for each value's tag.  Every rank must make the same sequence of calls on a
 * context, from one stream at a time.  A wait that runs out sets a fault (sm100_allreduce_fault != 0) and the kernel
 * returns; it never spins without bound. */
typedef void * sm100_allreduce_t;
SM100_API size_t sm100_ipc_handle_bytes(void);
SM100_API int sm100_ipc_export(void * device_ptr, void * handle_out);
SM100_API int sm100_ipc_open(const void * handle, void ** device_ptr_out);
SM100_API int sm100_ipc_close(void * device_ptr);
SM100_API size_t sm100_allreduce_area_bytes(int world, int capacity_floats);
SM100_API int sm100_allreduce_create(int rank, int world, int capacity_floats, void * const * areas, sm100_allreduce_t * out);
SM100_API int sm100_allreduce_sum(sm100_allreduce_t ctx, sm100_stream_t s, float * x, int n);
/* Greedy token over a vocabulary head whose rows are sharded over the ranks: x holds this rank's n logits (n may be 0),
 * index_offset the global index of x[0]; every rank receives in out[0] the global index of the largest logit of the whole
 * row, lowest index on ties (TOP_K with k = 1, src/core/ref/ops.cpp:1189-1228).  One single-CTA kernel per rank: local
 * arg-max, the (logit, index) candidates exchanged by tagged peer stores, bounded wait.  Every rank must call it the same
 * number of times.  The reference would copy every shard's logits to one device through the host and sort there. */
SM100_API int sm100_argmax_allreduce(sm100_allreduce_t ctx, sm100_stream_t s, const float * x, int64_t n, int64_t index_offset, int32_t * out);
SM100_API int sm100_allreduce_fault(sm100_allreduce_t ctx, int * fault_out);
/* polls (each followed by a sleep of about 0.1 us) before a wait for a peer gives up; default 1 << 22, about a second */
SM100_API int sm100_allreduce_set_wait_limit(sm100_allreduce_t ctx, uint32_t polls);
SM100_API int sm100_allreduce_destroy(sm100_allreduce_t ctx);
/* y[N] = sum over the ranks of W_r[K_r, N] . x_r[K_r]: the K-sharded ("row-parallel") product of tensor parallelism with
 * its all-reduce, M = 1; every rank calls it with its own shard and ends up with the same bits in y.  prologue 0: a is x;
 * SM100_PROLOGUE_SWIGLU: x = swiglu(a, b) (the down projection).  For packed Q4_K tensors with whole 16-row tiles the
 * exchange is folded into the matvec launch: every CTA stores the partial sums of its row tiles into its slot of every
 * rank's receive area (plain 8-byte peer stores: the value and the step number as its tag in one word, so neither a fence
 * nor a flag is needed) and adds the slots in rank order, waiting for each value's tag - bounded, about a second, after
 * which sm100_allreduce_fault reports it: the latency of one peer store at the end of the launch instead of a launch of
 * its own between two dependency boundaries.  Other tensors
 * run the matvec and sm100_allreduce_sum one after the other (same result contract).  All ranks must make the same
 * sequence of calls with the same shapes.  Like sm100_allreduce_sum it stands where the reference bounces through the
 * host (src/core/transport.cpp:53-146); the reference has no collective. */
SM100_API int sm100_mul_mat_allreduce(sm100_allreduce_t ctx, sm100_stream_t s, int prologue, const float * a, const float * b, int dtype,
                                      int layout, const void * w, int64_t k, int64_t n, float * y);

/* ---- timing and replay: the plan seat of the reference (src/core/registry.cpp:200-220, "selection
 *      happens once at plan build") becomes a captured CUDA graph ---- */
SM100_API int sm100_event_create(sm100_event_t * out);
SM100_API int sm100_event_destroy(sm100_event_t e);
SM100_API int sm100_event_record(sm100_event_t e, sm100_stream_t s);
/* work enqueued on s after this call starts only when the work recorded in e has completed (the backend's streams
 * are in-order, include/scrapgpu/stream.h:10-12; this is the edge between two of them: copies on one, kernels on another) */
SM100_API int sm100_stream_wait_event(sm100_stream_t s, sm100_event_t e);
SM100_API int sm100_event_sync(sm100_event_t e);
SM100_API int sm100_event_elapsed_ms(sm100_event_t start, sm100_event_t stop, float * ms);
SM100_API int sm100_graph_begin(sm100_stream_t s);
SM100_API int sm100_graph_end(sm100_stream_t s, sm100_graph_t * out);
SM100_API int sm100_graph_launch(sm100_graph_t g, sm100_stream_t s);
SM100_API int sm100_graph_destroy(sm100_graph_t g);
/* Library-owned scratch (slot 0 attention partials, 1 GEMM activation image, 2 quantized columns of the 3..8-column
 * matvec) is allocated on first use and only ever grows: a block that was handed out is never freed or moved, so CUDA
 * graphs captured earlier stay valid when a later, larger call makes the library allocate a bigger block.  Allocation
 * is impossible during stream capture; a caller that captures reserves the largest size it will need beforehand, either
 * by issuing the call once outside the capture or with sm100_scratch_reserve on the device in question.  No
 * counterpart in the reference (its backends allocate per call: src/core/attention.cpp:576). */
SM100_API int sm100_scratch_reserve(int slot, size_t bytes);
/* number of kernels of this library launched (or captured) by the calling process so far */
SM100_API uint64_t sm100_launch_count(void);
/* 1: launch kernels with programmatic dependent launch so that a kernel's weight prefetch overlaps
 * the tail of its predecessor on the same stream (default 1) */
SM100_API int sm100_set_pdl(int enabled);
/* What a kernel of this library may touch before its dependency wait, i.e. while kernels enqueued earlier on the
 * stream are still running: the WEIGHTS of the matvec / mul_mat / gemm entries (w, ws[i]) and nothing else.  Some
 * kernels release their successor before their own dependency wait, so "earlier" can reach back over several launches, up
 * to the last point of full serialization on the stream (a copy, an event wait, a graph launch, a synchronisation, a
 * kernel launched under sm100_launch_serialized).  A caller whose weight operand was produced by a kernel since that
 * point (a K cache used as the left operand, a weight converted on the device) brackets the call with
 * sm100_launch_serialized(1) ... (0): launches of the calling thread in between start only after everything enqueued
 * before them has completed.  sm100_pack_device needs no bracket: its kernel holds its successor back itself. */
SM100_API int sm100_launch_serialized(int on);

/* ---- weight packing: replaces the R32 repack of the OpenCL backend
 *      (src/backends/opencl11/r32.h:35-90, r32.cpp:19-86; geometry src/tensor/tensor.cpp:5-19).
 *      A packed tensor occupies exactly the natural byte count; packing is a byte permutation
 *      (plus a lossless re-encoding of the Q4_K 6-bit scale fields), so unpack(pack(w)) == w. ---- */
SM100_API size_t sm100_row_bytes(int dtype, int64_t k);                       /* src/tensor/tensor.h:54-66 */
SM100_API int sm100_pack(int dtype, int64_t k, int64_t n, const void * natural, void * packed);   /* host -> host */
SM100_API int sm100_unpack(int dtype, int64_t k, int64_t n, const void * packed, void * natural); /* host -> host */
/* device-side repack of a natural tensor already in HBM (src = natural, dst = packed, distinct buffers) */
SM100_API int sm100_pack_device(sm100_stream_t s, int dtype, int64_t k, int64_t n, const void * natural, void * packed);
SM100_API int sm100_unpack_device(sm100_stream_t s, int dtype, int64_t k, int64_t n, const void * packed, void * natural);
/* partial transfers on block boundaries (the chunked R32 transfer of src/backends/opencl11/r32.cpp:56-70):
 * `natural_chunk` holds blocks [first_block, first_block + block_count) of the tensor; to_packed != 0 scatters
 * them into the packed tensor at `packed`, 0 gathers them back */
SM100_API int sm100_pack_device_range(sm100_stream_t s, int dtype, int64_t k, int64_t n, int64_t first_block, int64_t block_count,
                                      void * natural_chunk, void * packed, int to_packed);

/* ---- the hot path: quantized MUL_MAT (src/core/ref/ops.cpp:891-984 exec_mul_mat; OpenCL kernels
 *      mul_mv_r.cl:240-323, mul_mv_k.cl:396-486, mul_mm.cl:271).  w, x, y are device pointers;
 *      x column stride ldx and y column stride ldy are in floats; w_row_stride is the byte stride of
 *      natural-layout weight rows (0 = dense; packed tensors are always dense).  m <= 8 takes the fused
 *      dequantize-and-dot matvec; larger m takes the tensor-core GEMM. ---- */
SM100_API int sm100_mul_mat(sm100_stream_t s, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k,
                            int64_t n, const float * x, int64_t ldx, int64_t m, float * y, int64_t ldy);
/* Name of the kernel family that served the calling thread's last sm100_mul_mat with m <= 8 ("matvec_q4k_imma",
 * "matvec_wide", "matvec_rows", ...; "+rows" when leftover rows took the row kernel).  The reference reports its kernel
 * choice per op key in its profile table (src/backends/opencl11/executor.h:41-112); here the parity tests use it to
 * prove that every branch of the dispatcher is exercised. */
SM100_API const char * sm100_matvec_last_kernel(void);
/* MUL_MAT with activations and results in HOST memory, one call per product and no host synchronisation in between:
 * what a caller of the reference does with scrapgpu_tensor_upload -> op_execute -> scrapgpu_tensor_download
 * (include/scrapgpu/tensor.h:45-53), as a pipeline.  A pipe owns three in-order streams and `depth` slots of device
 * staging (max_x_bytes of activations, max_y_bytes of results each): the copy of the next product's activations and
 * the read-back of the previous product's result run beside the current product's kernel.  host_x [k * m] and
 * host_y [n * m] are dense f32 (column stride k and n); they must stay untouched until sm100_hostpipe_sync returns,
 * and should be pinned (sm100_host_alloc) so that the copies overlap.  w is a device pointer as for sm100_mul_mat.
 * sm100_hostpipe_stream hands out the pipe's streams (0 copy-in, 1 kernels, 2 read-back), e.g. to time a region with
 * events.  One pipe is used from one thread at a time.  These entries have no counterpart in the reference. */
typedef struct sm100_hostpipe_s * sm100_hostpipe_t;
SM100_API int sm100_hostpipe_create(int device, int depth, size_t max_x_bytes, size_t max_y_bytes, sm100_hostpipe_t * out);
SM100_API int sm100_hostpipe_destroy(sm100_hostpipe_t pipe);
SM100_API int sm100_hostpipe_stream(sm100_hostpipe_t pipe, int which, sm100_stream_t * out);
SM100_API int sm100_hostpipe_mul_mat(sm100_hostpipe_t pipe, int dtype, int layout, const void * w, int64_t w_row_stride,
                                     int64_t k, int64_t n, const float * host_x, int64_t m, float * host_y);
/* the same for a list of products (a plan's worth, include/scrapgpu/backend.h:29-57 plan_execute): one call enqueues
 * them all in order; returns at the first failing item */
typedef struct sm100_hostpipe_item {
    int dtype, layout;
    const void * w;          /* device */
    int64_t w_row_stride, k, n;
    const float * host_x;
    int64_t m;
    float * host_y;
} sm100_hostpipe_item;
SM100_API int sm100_hostpipe_mul_mat_many(sm100_hostpipe_t pipe, int count, const sm100_hostpipe_item * items);
SM100_API int sm100_hostpipe_sync(sm100_hostpipe_t pipe);
/* MUL_MAT_MULTI (include/scrapgpu/op.h:46, src/backends/opencl11/kernels/mul_mv_multi.cl:46-104):
 * up to 3 weight tensors sharing one activation column, one launch */
SM100_API int sm100_mul_mat_multi(sm100_stream_t s, int count, const int * dtypes, const int * layouts,
                                  const void * const * ws, int64_t k, const int64_t * ns, const float * x,
                                  float * const * ys);

/* MUL_MAT_MULTI with the producer of the activation column folded into the same launch (one f32 column).
 *   SM100_PROLOGUE_SWIGLU    x = swiglu(a, b) = (a / (1 + expf(-a))) * b                 (src/core/ref/ops.cpp:383-425)
 *   SM100_PROLOGUE_RMS_NORM  s = a (+ b when b != NULL), x = rms_norm(s, eps) * norm_w   (RMS_NORM_MUL / ADD_RMS_NORM_MUL,
 *                            include/scrapgpu/op.h:43-44, src/core/ref/ops.cpp:466-519); s is written to sum_out and
 *                            x to x_out when those are non-NULL; they must not alias a or b
 * Same values as the separate ops followed by sm100_mul_mat_multi.  Served for packed Q4_K tensors whose row counts
 * are multiples of 16 (K a multiple of 256, at most 8192 for the norm); otherwise UNSUPPORTED (status 1) and the
 * caller runs the separate ops. */
#define SM100_PROLOGUE_SWIGLU 1
#define SM100_PROLOGUE_RMS_NORM 2
/* The gate and up projections of a gated FFN with their SwiGLU in ONE launch: act = swiglu(W_gate . x, W_up . x), where x is
 * `a` (prologue 0) or the (ADD_)RMS_NORM_MUL row of sm100_mul_mat_fused (SM100_PROLOGUE_RMS_NORM, with the same sum_out /
 * x_out side outputs).  The kernel walks the row tiles of the two tensors alternately, so a CTA holds row i of gate and of up
 * at the same time and writes the activation directly: the down projection that follows is a plain matvec, without a SwiGLU
 * kernel in front of it and without every one of its CTAs evaluating SwiGLU over the whole row.  gate_out / up_out (optional)
 * receive the projections themselves.  Same values as MUL_MAT_MULTI followed by GLU (include/scrapgpu/op.h:46, src/core/ref/ops.cpp:383-425).
 * Packed Q4_K tensors [K, N] with N a multiple of 16; otherwise UNSUPPORTED (status 1) and the caller runs the separate ops. */
SM100_API int sm100_mul_mat_glu(sm100_stream_t s, int prologue, const float * a, const float * b, const float * norm_w, float eps,
                                float * sum_out, float * x_out, int dtype, int layout, const void * w_gate, const void * w_up,
                                int64_t k, int64_t n, float * gate_out, float * up_out, float * act_out);
SM100_API int sm100_mul_mat_fused(sm100_stream_t s, int prologue, const float * a, const float * b, const float * norm_w,
                                  float eps, float * sum_out, float * x_out, int count, const int * dtypes,
                                  const int * layouts, const void * const * ws, int64_t k, const int64_t * ns,
                                  float * const * ys);

/* ---- bit-exact dequantization: GET_ROWS over a quantized / F32 / F16 table
 *      (src/core/ref/ops.cpp:690-722, quant.cpp:30-108); ids are I32 on the device; table_row_stride is the
 *      byte stride of natural-layout rows (0 = dense) ---- */
SM100_API int sm100_get_rows(sm100_stream_t s, int dtype, int layout, const void * table, int64_t table_row_stride,
                             int64_t k, int64_t table_rows, const int32_t * ids, int64_t n_ids, float * dst,
                             int64_t ld_dst);

/* ---- the ops around the matvec in a decode step ---- */
/* RMS_NORM / RMS_NORM_MUL / ADD_RMS_NORM_MUL (ops.cpp:440-519): add, w, sum_out may be NULL */
SM100_API int sm100_rms_norm(sm100_stream_t s, const float * x, const float * add, const float * w, float * sum_out,
                             float * y, int64_t ne0, int64_t rows, float eps);
/* ROPE (ops.cpp:530-634) with a (cos, sin) table [n_positions, n_dims/2, 2] computed by the caller the
 * way the reference does (sequential theta products, libm cos/sin); positions are I32 on the device and
 * index the table after subtracting table_first_position */
SM100_API int sm100_rope(sm100_stream_t s, const float * x, const int32_t * positions, const float * table,
                         int32_t table_first_position, int32_t table_positions, float * y, int64_t ne0,
                         int64_t heads, int64_t tokens, int n_dims, int neox);
/* ROPE computing cos/sin on the device (sequential theta products in f32, cosf/sinf) */
SM100_API int sm100_rope_direct(sm100_stream_t s, const float * x, const int32_t * positions, float * y, int64_t ne0,
                                int64_t heads, int64_t tokens, int n_dims, int neox, float freq_base, float freq_scale,
                                float attn_factor);
/* SOFT_MAX (ops.cpp:636-684): y = softmax(x*scale + mask) per row; mask may be NULL; in place allowed */
SM100_API int sm100_soft_max(sm100_stream_t s, const float * x, const float * mask, int64_t mask_row_stride,
                             float * y, int64_t ne0, int64_t rows, float scale);
/* GLU SwiGLU with split inputs (ops.cpp:383-425) */
SM100_API int sm100_swiglu(sm100_stream_t s, const float * x, const float * g, float * y, int64_t n);
/* ADD, same shapes (ops.cpp:280-312) */
SM100_API int sm100_add(sm100_stream_t s, const float * a, const float * b, float * y, int64_t n);
/* SET_ROWS F32 -> F32 (ops.cpp:724-762): dst[:, ids[i], h] = src[:, i, h] */
SM100_API int sm100_set_rows(sm100_stream_t s, const float * src, const int32_t * ids, float * dst, int64_t ne0,
                             int64_t n_rows, int64_t heads, int64_t dst_rows);
/* One decode token's head post-processing in one launch: RMS_NORM_MUL per head of Q and K (weights may be NULL: no
 * norm), ROPE of Q and K (full head rotated; NEOX or NORMAL pairing; (cos, sin) from the table, positions outside
 * it take the on-device recipe), and SET_ROWS_PAIR of K and V into the caches [kv_heads][cache_rows][head_dim]
 * (include/scrapgpu/op.h:43-45 RMS_NORM_MUL / SET_ROWS_PAIR, src/core/ref/ops.cpp:440-519, 530-634, 690-760).
 * Same values as the separate ops; Q and K are updated in place; positions is one I32 on the device. */
SM100_API int sm100_head_post(sm100_stream_t s, float * q, float * k, const float * v, const float * q_norm_w,
                              const float * k_norm_w, const int32_t * positions, const float * table,
                              int32_t table_first_position, int32_t table_positions, float * k_cache, float * v_cache,
                              int64_t head_dim, int64_t q_heads, int64_t kv_heads, int64_t cache_rows, float eps,
                              float freq_base, int neox);

/* sm100_head_post followed by sm100_attention_kvcache (one query, causal over the cache up to positions[0], fresh_keys 1) for
 * one decode token - in ONE launch where the shapes allow (NEOX rotation, head_dim 128 or 256, 1 / 2 / 4 / 8 query heads per KV
 * head, a cache short enough for the single-launch merge): every warp of the attention kernel normalises and rotates the
 * query heads it uses, the CTA whose split ends at the newest position does the same for the new key, stores it and the new
 * value into the caches and reads them back like any other row.  Other shapes run the two launches.  Same arguments as
 * sm100_head_post plus the attention output [head_dim, q_heads] and the score scale; unlike sm100_head_post it leaves q and
 * k_new as they were in the single-launch form (nothing else may rely on them being rotated in place).  Values: those of the
 * two separate calls up to the order of the double-precision additions in the norms' sums of squares. */
SM100_API int sm100_attention_decode(sm100_stream_t s, float * q, float * k_new, const float * v_new, const float * q_norm_w,
                                     const float * k_norm_w, const int32_t * positions, const float * table,
                                     int32_t table_first_position, int32_t table_positions, float * k_cache, float * v_cache,
                                     float * out, int64_t head_dim, int64_t q_heads, int64_t kv_heads, int64_t cache_rows, float eps,
                                     float freq_base, int neox, float scale);

/* TOP_K with k = 1 (ops.cpp:1189-1228): index of the maximum, lowest index on ties */
SM100_API int sm100_argmax(sm100_stream_t s, const float * x, int64_t n, int32_t * out);
/* fused decode attention, the values of scrapgpu_scaled_dot_product_attention
 * (src/core/attention.cpp:558-678, include/scrapgpu/attention.h:11-46): Q [D, nq, Hq], K [D, nk, Hkv],
 * V [Dv, nk, Hkv], out [Dv, nq, Hq], causal rule k <= offset + q.  mask (optional) is additive F32
 * [nk, nq, mask_heads] with mask_heads 1 or Hq.  When positions is non-NULL the offset is read from
 * positions[0] on the device instead of the argument, so one captured graph serves every step.
 * Uses a per-device scratch buffer owned by the library (allocated on first use: make the first call
 * outside stream capture). */
SM100_API int sm100_attention(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask,
                              int64_t mask_heads, float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk, int64_t hq,
                              int64_t hkv, int causal, int64_t offset, const int32_t * positions, float scale);

/* sm100_attention over a KV cache, with one promise from the caller that lets the key/value rows be requested while
 * launches that precede this call in the stream are still running: of each query's visible keys only the last
 * fresh_keys (>= 0) may have been written since the stream's last point of full serialization (a copy, an event wait,
 * a graph launch, a synchronisation, a kernel launched without programmatic dependent launch: see
 * sm100_launch_serialized); every earlier K/V row, and positions[0], were written before that point.  In a decode
 * step the promise holds with fresh_keys = 1: the step stores the new token's K and V (SET_ROWS / SET_ROWS_PAIR,
 * include/scrapgpu/op.h:43-47) and all older rows date from earlier steps, which a graph launch or the host's read
 * of the token separates from this one.  Same values as sm100_attention; with the promise broken the result is
 * undefined.  This entry has no counterpart in the reference. */
SM100_API int sm100_attention_kvcache(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask,
                                      int64_t mask_heads, float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk,
                                      int64_t hq, int64_t hkv, int causal, int64_t offset, const int32_t * positions,
                                      float scale, int fresh_keys);

/* sm100_attention for callers that cannot allocate device memory at call time (a host whose HBM is fully claimed
 * by its own pools, a latency-critical thread that must stay off the driver's allocator, an externally enforced
 * memory budget).  Same arguments and values as sm100_attention; the split-key partials go to a fixed 4 MiB array
 * inside the library image (every GPU that loads the library holds it until exit) instead of a scratch buffer
 * allocated on demand.  sm100_attention_static_capacity() is the array's size; its first 64 KiB hold the ticket
 * counters of the single-launch merge, so shapes whose partials (nq * hq * splits * (dv + 4) floats) exceed the
 * capacity minus 64 KiB are refused with UNSUPPORTED.  The first call on a device looks the array's address up:
 * make it before any stream capture.  All calls on one device share the array and it keeps the last call's
 * contents: every call first clears the counters it will use (a memset on the caller's stream, no allocation), the
 * partials need no clearing; calls that overlap on the GPU race, and a raced call's result is undefined (later,
 * non-overlapping calls are correct again because of the clearing).  This entry has no counterpart in the reference. */
SM100_API int sm100_attention_static(sm100_stream_t s, const float * q, const float * k, const float * v, const float * mask,
                                     int64_t mask_heads, float * out, int64_t d, int64_t dv, int64_t nq, int64_t nk,
                                     int64_t hq, int64_t hkv, int causal, int64_t offset, const int32_t * positions,
                                     float scale);
SM100_API size_t sm100_attention_static_capacity(void);
/* Does, for the current device, the one-time address look-up that the first sm100_attention_static call on a device
 * would otherwise do, so that a caller can get it out of the way explicitly before it starts a stream capture; allocates
 * nothing.  device_address_out (may be NULL) receives the array's device address, for diagnostics only: the contents
 * belong to the library.  No counterpart in the reference. */
SM100_API int sm100_attention_static_prepare(void ** device_address_out);

/* ---- the same ops over strided views (arbitrary nb[1..3], broadcast operands, transposed CPY sources): what
 *      op_execute needs to honour every descriptor the reference's CPU backend accepts
 *      (src/backends/cpu/api.cpp:394-830) ---- */
SM100_API int sm100_binary(sm100_stream_t s, int op /* 0 ADD 1 SUB 2 MUL 3 DIV */, const sm100_view * a, const sm100_view * b,
                           const sm100_view * y);                                          /* ops.cpp:280-312 */
SM100_API int sm100_glu(sm100_stream_t s, int kind /* 0 SwiGLU 1 ReGLU */, const sm100_view * x, const sm100_view * g /* NULL: fused halves */,
                        int swapped, const sm100_view * y);                                 /* ops.cpp:383-425 */
SM100_API int sm100_rms_norm_view(sm100_stream_t s, const sm100_view * x, const sm100_view * add, const float * w,
                                  const sm100_view * sum_out, const sm100_view * y, float eps); /* ops.cpp:440-519 */
SM100_API int sm100_rope_view(sm100_stream_t s, const sm100_view * x, const int32_t * positions, const float * table,
                              int32_t table_first_position, int32_t table_positions, const float * freq_factors,
                              const sm100_view * y, int n_dims, int neox, float freq_base, float freq_scale,
                              float attn_factor);                                           /* ops.cpp:530-634 */
/* the same for F16 tensors (x and y share the dtype, ops.cpp:531-533): dtype is 0 (F32) or 1 (F16) */
SM100_API int sm100_rope_view_dt(sm100_stream_t s, int dtype, const sm100_view * x, const int32_t * positions, const float * table,
                                 int32_t table_first_position, int32_t table_positions, const float * freq_factors,
                                 const sm100_view * y, int n_dims, int neox, float freq_base, float freq_scale, float attn_factor);
/* SCALE / CLAMP / SQR / SQRT / UNARY over F32 views of one shape (ops.cpp:314-381).  code: 0 SCALE y = x * p0 + p1,
 * 1 CLAMP to [p0, p1], 2 SQR, 3 SQRT, 10 + scrapgpu_unary_kind (include/scrapgpu/op.h:50-57: SILU, RELU, NEG, ABS,
 * SIGMOID, TANH) */
SM100_API int sm100_unary(sm100_stream_t s, int code, float p0, float p1, const sm100_view * x, const sm100_view * y);
SM100_API int sm100_soft_max_view(sm100_stream_t s, const sm100_view * x, const sm100_view * mask, int mask_is_f16,
                                  const sm100_view * y, float scale);                       /* ops.cpp:636-684 */
SM100_API int sm100_cpy(sm100_stream_t s, const sm100_view * src, int src_dtype, const sm100_view * dst, int dst_dtype); /* ops.cpp:764-800 */
SM100_API int sm100_set_rows_view(sm100_stream_t s, const sm100_view * src, int src_dtype, const sm100_view * ids, int ids_are_i64,
                                  const sm100_view * dst, int dst_dtype);                   /* ops.cpp:724-762 */
SM100_API int sm100_top1_view(sm100_stream_t s, const sm100_view * x, const sm100_view * out);   /* ops.cpp:1189-1228, k = 1 */
/* CONT_MUL_MAT (include/scrapgpu/op.h:47; inputs [a, x] per src/backends/opencl11/api.cpp:11-12; OpenCL kernels
 * attn.cl:123-237): `a` is the transposed F16 (or F32) view a CONT would have copied -- its dim 1 is the contiguous
 * one -- and dst[i1, 0, i2, i3] = sum_i0 a[i0, i1, i2 / r2, i3 / r3] * x[i0, 0, i2, i3], the values of CONT followed
 * by MUL_MAT (src/core/ref/ops.cpp:764-800, 891-984) without the copy */
SM100_API int sm100_cont_mul_mat(sm100_stream_t s, const sm100_view * a, int a_dtype, const sm100_view * x, const sm100_view * y);

#ifdef __cplusplus
}
#endif

#endif
