/* Link-time shim for callers that name their backend in source.  The reference's
 * examples/standalone_matmul.c:67 calls scrapgpu_opencl11_register(); linked against this object instead of the
 * OpenCL backend, the byte-for-byte unchanged example runs on cuda_sm100.  Only legal where the OpenCL backend is
 * not linked into the same program. */
#include "scrapgpu/cuda_sm100.h"

SCRAPGPU_API scrapgpu_status scrapgpu_opencl11_register(void) { return scrapgpu_cuda_sm100_register(); }
