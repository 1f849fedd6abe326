/*
 * scrapgpu/cuda_sm100.h -- the one public header the `cuda_sm100` backend adds to ScrapGpuLibrary.
 *
 * The backend registers through the existing registry (scrapgpu_register_backend,
 * include/scrapgpu/backend.h:59) exactly like the CPU / OpenCL / Vulkan backends do
 * (include/scrapgpu/cpu.h:16, include/scrapgpu/opencl11.h, include/scrapgpu/vulkan.h:11-16); after that the
 * unchanged scrapgpu_ device / buffer / stream / plan / op API drives B200 GPUs.
 *
 * Layout tag: quantized weights uploaded with SCRAPGPU_LAYOUT_R32 (the "backend-packed" tag existing callers
 * already pass for GPU backends) are stored in the B200 plane layout; the host always sees natural GGUF bytes.
 */
#ifndef SCRAPGPU_CUDA_SM100_H
#define SCRAPGPU_CUDA_SM100_H

#include "scrapgpu/attention.h"
#include "scrapgpu/backend.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Registers the backend "cuda_sm100": one device per visible CUDA GPU of compute capability 10.x.
 * Idempotent and thread-safe; succeeds with zero devices when no such GPU is present.  Fails with
 * SCRAPGPU_STATUS_UNSUPPORTED when the ScrapGpuLibrary core is not loaded in the process. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_register(void);

/* The backend's vtable (ABI 0.4), usable without the registry: every object it hands out carries it in its
 * scrapgpu_object_header. */
SCRAPGPU_API const scrapgpu_backend_vtable * scrapgpu_cuda_sm100_vtable(void);

/* scrapgpu_scaled_dot_product_attention (include/scrapgpu/attention.h:11-46) as ONE fused kernel pair on a
 * cuda_sm100 device: same tensors, same causal / mask / GQA rules, same values within float rounding.  The
 * core entry keeps working on this backend through its CPY + MUL_MAT + SOFT_MAX composition; this entry is the
 * fast path for decode (the vtable has no attention slot). */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_attention(scrapgpu_device_t * device, scrapgpu_stream_t * stream,
                                                          const scrapgpu_attention_params * params);
/* As above, but the causal offset is read on the device from an I32 tensor (first element) when the stream
 * reaches the call, so a recorded plan or graph can be replayed for successive positions. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_attention_at(scrapgpu_device_t * device, scrapgpu_stream_t * stream,
                                                             const scrapgpu_attention_params * params,
                                                             const scrapgpu_tensor_desc * position);

/* ---- multi-GPU transport -----------------------------------------------------------------------------------------
 * The core moves a tensor between two devices through a host staging buffer: a blocking read on the source stream,
 * then a blocking write on the destination stream (src/core/transport.cpp:128-145, contract
 * include/scrapgpu/tensor.h:55-67).  Between two cuda_sm100 devices the bytes can go GPU to GPU over NVLink instead. */

/* scrapgpu_tensor_copy for two cuda_sm100 tensors: same contract (contiguous tensors of one dtype and shape, natural
 * layout only, the copy happens after the work already enqueued on src_stream and before work enqueued later on
 * dst_stream), but asynchronous and without the host bounce: an event on src_stream, a wait on dst_stream, one
 * peer copy.  Works for the same device too. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_tensor_copy(scrapgpu_stream_t * src_stream, const scrapgpu_tensor_desc * src,
                                                            scrapgpu_stream_t * dst_stream, const scrapgpu_tensor_desc * dst);

/* A group of cuda_sm100 devices that run one model tensor-parallel from ONE process (one stream per device, each
 * driven by the calling thread as the contract asks, docs/API_CONTRACT.md:59).  Creating the group enables peer access
 * between all pairs and sets up the receive areas of the one-shot all-reduce (up to 8 devices, max_elements floats). */
typedef struct scrapgpu_cuda_sm100_group scrapgpu_cuda_sm100_group_t;
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_create(scrapgpu_device_t * const * devices, size_t count, size_t max_elements,
                                                             scrapgpu_cuda_sm100_group_t ** out_group);
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_free(scrapgpu_cuda_sm100_group_t * group);
/* In-place sum over the group: tensors[i] (F32, contiguous, the same length on every device, a multiple of 4 elements,
 * 16-byte aligned) lives on device i and is updated on streams[i]; every device ends up with the same bits (the
 * partial vectors are added in device order).  One kernel per device; a device that waits longer than about a second
 * for a peer gives up and the next scrapgpu_cuda_sm100_group_status reports BACKEND_ERROR. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_all_reduce(scrapgpu_cuda_sm100_group_t * group, scrapgpu_stream_t * const * streams,
                                                                 const scrapgpu_tensor_desc * tensors);
/* The row-parallel product of tensor parallelism with its all-reduce: outputs[i] (F32 [N], the same N everywhere) on every
 * device receives the sum over the devices of weights[i] [K_i, N] . inputs[i] [K_i], the same bits everywhere.  weights[i] is
 * device i's K shard (scrapgpu_cuda_sm100_shard with split_dim 0, uploaded with scrapgpu_cuda_sm100_upload_view).  For packed
 * Q4_K shards with whole 16-row tiles the exchange happens inside the matvec launch of every device (peer stores tagged
 * with the step number, bounded waits: see scrapgpu_cuda_sm100_group_status); other tensors run MUL_MAT and
 * scrapgpu_cuda_sm100_group_all_reduce one after the other.  In the core's terms this is MUL_MAT on every device followed
 * by the tensor copies and ADDs that src/core/transport.cpp:53-146 would bounce through the host. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_mul_mat_all_reduce(scrapgpu_cuda_sm100_group_t * group, scrapgpu_stream_t * const * streams,
                                                                         const scrapgpu_tensor_desc * weights, const scrapgpu_tensor_desc * inputs,
                                                                         const scrapgpu_tensor_desc * outputs);
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_group_status(scrapgpu_cuda_sm100_group_t * group);

/* Shard arithmetic for tensor parallelism, on descriptors only (no device needed).  `full` describes a natural-layout
 * 2-D weight [K, N] (N rows of K elements); out_view receives the view of rank `rank` of `world`:
 *   split_dim 1 (column-parallel: Q, K, V, gate, up, vocabulary head): rows [rank * ceil(N / world), ...), the last
 *               rank may get fewer rows (or none: ne[1] = 0);
 *   split_dim 0 (row-parallel: o, down): elements [rank * K / world, (rank + 1) * K / world) of every row; K / world
 *               must be a whole number of quantization blocks.  The view keeps the row stride of the full tensor.
 * The view shares `full`'s buffer field and has offset advanced accordingly, so it describes the shard inside a host
 * image of the full tensor just as well as inside a device buffer. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_shard(const scrapgpu_tensor_desc * full, int split_dim, size_t rank, size_t world,
                                                      scrapgpu_tensor_desc * out_view);
/* Uploads the (possibly strided) view `src_view` of a natural-layout host image starting at `host_base` (the byte the
 * view's offset counts from) into the contiguous device tensor `dst` of the same dtype and shape; dst may carry the
 * packed-layout tag.  This is tensor_upload for a shard cut out of the full tensor's host image. */
SCRAPGPU_API scrapgpu_status scrapgpu_cuda_sm100_upload_view(scrapgpu_stream_t * stream, const scrapgpu_tensor_desc * dst, const void * host_base,
                                                            const scrapgpu_tensor_desc * src_view);

/* Kernels launched by this process through the backend so far (per-process counter for profiling). */
SCRAPGPU_API uint64_t scrapgpu_cuda_sm100_launch_count(void);

/* The per-op-key timing table, the counterpart of the OpenCL backend's GGML_CL11_PROFILE table
 * (src/backends/opencl11/executor.h:41-112; keys as adapters/ggml/ggml-cl11.cpp:1033-1049).  With the environment
 * variable SCRAPGPU_SM100_PROFILE=1 every op executed on a stream (directly or as a plan step; plans then run step by
 * step instead of replaying a graph, and every launch is fully serialized) is bracketed by two events; stream_sync
 * adds the finished pairs to the stream's table, stream_free prints it to stderr.  This call writes the table collected
 * so far ("<key> <calls> <ms> <us/call> <share> [weights GB/s]", slowest first) into out (NUL-terminated, truncated to
 * capacity) and returns the size the whole text needs, 0 when the table is off or empty.
 * SCRAPGPU_SM100_PROFILE_SHAPES=1 adds the shape of src0 to the keys. */
SCRAPGPU_API size_t scrapgpu_cuda_sm100_profile_report(scrapgpu_stream_t * stream, char * out, size_t capacity);

#ifdef __cplusplus
}
#endif

#endif
