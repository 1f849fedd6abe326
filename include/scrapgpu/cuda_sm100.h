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

/* Kernels launched by this process through the backend so far (per-process counter for profiling). */
SCRAPGPU_API uint64_t scrapgpu_cuda_sm100_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif
