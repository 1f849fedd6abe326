// Host and device packing between natural GGUF blocks and the B200 plane layout (sm100_layout.h).
// Stands in for the OpenCL backend's R32 repack (src/backends/opencl11/r32.h:35-90, r32.cpp:19-86 of
// the reference) with the same contract: the host always sees natural bytes, the packed tensor has
// the natural size, unpack(pack(w)) == w byte for byte.
#include "sm100_common.cuh"
#include "sm100_layout.h"

#include <cstring>

namespace sm100 {

// One block, natural -> packed.  `dst` is the tensor base of the packed image, t the block number.
__host__ __device__ inline void pack_block(int dtype, const Planes & P, int64_t t, const uint8_t * blk, uint8_t * dst) {
    if (dtype == DT_Q4_K) {
        uint8_t * h = dst + P.off[1] + t * 16;
        const int64_t row = t / P.blocks_per_row, b = t % P.blocks_per_row;
        for (int i = 0; i < 128; ++i) dst[P.off[0] + q4k_q_offset(P, row, b, i)] = blk[16 + i];
        h[0] = blk[0]; h[1] = blk[1]; h[2] = blk[2]; h[3] = blk[3];
        const uint8_t * s = blk + 4;
        for (int p = 0; p < 4; ++p) {
            uint32_t sc[2], mn[2];
            for (int e = 0; e < 2; ++e) {
                const int j = 2 * p + e;
                if (j < 4) {
                    sc[e] = s[j] & 63u;
                    mn[e] = s[j + 4] & 63u;
                } else {
                    sc[e] = (s[j + 4] & 15u) | ((uint32_t) (s[j - 4] >> 6) << 4);
                    mn[e] = (uint32_t) (s[j + 4] >> 4) | ((uint32_t) (s[j] >> 6) << 4);
                }
            }
            const uint32_t f = sc[0] | (mn[0] << 6) | (sc[1] << 12) | (mn[1] << 18);
            h[4 + 3 * p + 0] = (uint8_t) (f & 255u);
            h[4 + 3 * p + 1] = (uint8_t) ((f >> 8) & 255u);
            h[4 + 3 * p + 2] = (uint8_t) ((f >> 16) & 255u);
        }
    } else if (dtype == DT_Q6_K) {
        uint8_t * l = dst + P.off[0] + t * 128;
        uint8_t * x = dst + P.off[1] + t * 64;
        uint8_t * s = dst + P.off[2] + t * 16;
        uint8_t * d = dst + P.off[3] + t * 2;
        for (int h = 0; h < 2; ++h)
            for (int c = 0; c < 2; ++c) {
                const int u = 2 * h + c;
                for (int i = 0; i < 16; ++i) {
                    l[32 * u + i] = blk[64 * h + 16 * c + i];
                    l[32 * u + 16 + i] = blk[64 * h + 32 + 16 * c + i];
                }
                for (int g = 0; g < 4; ++g) s[4 * u + g] = blk[192 + 8 * h + c + 2 * g];
            }
        for (int i = 0; i < 64; ++i) x[i] = blk[128 + i];
        d[0] = blk[208];
        d[1] = blk[209];
    } else if (dtype == DT_Q4_0) {
        uint8_t * q = dst + P.off[0] + t * 16;
        uint8_t * d = dst + P.off[1] + t * 2;
        for (int i = 0; i < 16; ++i) q[i] = blk[2 + i];
        d[0] = blk[0];
        d[1] = blk[1];
    } else if (dtype == DT_Q8_0) {
        uint8_t * q = dst + P.off[0] + t * 32;
        uint8_t * d = dst + P.off[1] + t * 2;
        for (int i = 0; i < 32; ++i) q[i] = blk[2 + i];
        d[0] = blk[0];
        d[1] = blk[1];
    }
}

// One block, packed -> natural.
__host__ __device__ inline void unpack_block(int dtype, const Planes & P, int64_t t, const uint8_t * src, uint8_t * blk) {
    if (dtype == DT_Q4_K) {
        const uint8_t * h = src + P.off[1] + t * 16;
        const int64_t row = t / P.blocks_per_row, b = t % P.blocks_per_row;
        for (int i = 0; i < 128; ++i) blk[16 + i] = src[P.off[0] + q4k_q_offset(P, row, b, i)];
        blk[0] = h[0]; blk[1] = h[1]; blk[2] = h[2]; blk[3] = h[3];
        uint32_t sc[8], mn[8];
        for (int p = 0; p < 4; ++p) {
            const uint32_t f = (uint32_t) h[4 + 3 * p] | ((uint32_t) h[5 + 3 * p] << 8) | ((uint32_t) h[6 + 3 * p] << 16);
            sc[2 * p] = f & 63u;
            mn[2 * p] = (f >> 6) & 63u;
            sc[2 * p + 1] = (f >> 12) & 63u;
            mn[2 * p + 1] = (f >> 18) & 63u;
        }
        uint8_t * s = blk + 4;
        for (int j = 0; j < 4; ++j) {
            s[j] = (uint8_t) (sc[j] | ((sc[j + 4] >> 4) << 6));
            s[j + 4] = (uint8_t) (mn[j] | ((mn[j + 4] >> 4) << 6));
            s[j + 8] = (uint8_t) ((sc[j + 4] & 15u) | ((mn[j + 4] & 15u) << 4));
        }
    } else if (dtype == DT_Q6_K) {
        const uint8_t * l = src + P.off[0] + t * 128;
        const uint8_t * x = src + P.off[1] + t * 64;
        const uint8_t * s = src + P.off[2] + t * 16;
        const uint8_t * d = src + P.off[3] + t * 2;
        for (int h = 0; h < 2; ++h)
            for (int c = 0; c < 2; ++c) {
                const int u = 2 * h + c;
                for (int i = 0; i < 16; ++i) {
                    blk[64 * h + 16 * c + i] = l[32 * u + i];
                    blk[64 * h + 32 + 16 * c + i] = l[32 * u + 16 + i];
                }
                for (int g = 0; g < 4; ++g) blk[192 + 8 * h + c + 2 * g] = s[4 * u + g];
            }
        for (int i = 0; i < 64; ++i) blk[128 + i] = x[i];
        blk[208] = d[0];
        blk[209] = d[1];
    } else if (dtype == DT_Q4_0) {
        const uint8_t * q = src + P.off[0] + t * 16;
        const uint8_t * d = src + P.off[1] + t * 2;
        for (int i = 0; i < 16; ++i) blk[2 + i] = q[i];
        blk[0] = d[0];
        blk[1] = d[1];
    } else if (dtype == DT_Q8_0) {
        const uint8_t * q = src + P.off[0] + t * 32;
        const uint8_t * d = src + P.off[1] + t * 2;
        for (int i = 0; i < 32; ++i) blk[2 + i] = q[i];
        blk[0] = d[0];
        blk[1] = d[1];
    }
}

// blocks [first, first + count): natural holds them contiguously starting at its byte 0
__global__ void pack_kernel(int dtype, Planes P, int64_t first, int64_t count, int bb, const uint8_t * natural, uint8_t * packed, int to_packed) {
    // never releases its successor early: what it writes are weights, which the matvec kernels request before their
    // own dependency wait
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < count; i += (int64_t) gridDim.x * blockDim.x) {
        if (to_packed) pack_block(dtype, P, first + i, natural + i * bb, packed);
        else unpack_block(dtype, P, first + i, packed, const_cast<uint8_t *>(natural) + i * bb);
    }
}

static int check_shape(int dtype, int64_t k, int64_t n, const char * who) {
    if (!is_quant(dtype)) return fail(ST_UNSUPPORTED, "%s: dtype %d has no packed layout", who, dtype);
    if (k <= 0 || n <= 0 || k % block_elems(dtype) != 0)
        return fail(ST_INVALID, "%s: K must be a positive multiple of the block size and N positive", who);
    return ST_OK;
}

}  // namespace sm100

using namespace sm100;

extern "C" {

size_t sm100_row_bytes(int dtype, int64_t k) {
    const int be = block_elems(dtype);
    if (be == 0 || k < 0) return 0;
    return (size_t) ((k + be - 1) / be) * (size_t) block_bytes(dtype);
}

int sm100_pack(int dtype, int64_t k, int64_t n, const void * natural, void * packed) {
    if (natural == nullptr || packed == nullptr) return fail(ST_INVALID, "sm100_pack: null pointer");
    const int st = check_shape(dtype, k, n, "sm100_pack");
    if (st != ST_OK) return st;
    const int64_t total = n * (k / block_elems(dtype));
    const Planes P = planes_for(dtype, n, k);
    const int bb = block_bytes(dtype);
    for (int64_t t = 0; t < total; ++t) pack_block(dtype, P, t, (const uint8_t *) natural + t * bb, (uint8_t *) packed);
    return ST_OK;
}

int sm100_unpack(int dtype, int64_t k, int64_t n, const void * packed, void * natural) {
    if (natural == nullptr || packed == nullptr) return fail(ST_INVALID, "sm100_unpack: null pointer");
    const int st = check_shape(dtype, k, n, "sm100_unpack");
    if (st != ST_OK) return st;
    const int64_t total = n * (k / block_elems(dtype));
    const Planes P = planes_for(dtype, n, k);
    const int bb = block_bytes(dtype);
    for (int64_t t = 0; t < total; ++t) unpack_block(dtype, P, t, (const uint8_t *) packed, (uint8_t *) natural + t * bb);
    return ST_OK;
}

static int pack_device(sm100_stream_t s, int dtype, int64_t k, int64_t n, int64_t first, int64_t count, const void * natural, void * packed,
                       int to_packed) {
    if (natural == nullptr || packed == nullptr) return fail(ST_INVALID, "sm100_pack_device: null pointer");
    const int st = check_shape(dtype, k, n, "sm100_pack_device");
    if (st != ST_OK) return st;
    const int64_t total = n * (k / block_elems(dtype));
    if (first < 0 || count < 0 || first + count > total) return fail(ST_INVALID, "sm100_pack_device: block range outside the tensor");
    if (count == 0) return ST_OK;
    const Planes P = planes_for(dtype, n, k);
    const int threads = 128;
    int64_t blocks = (count + threads - 1) / threads;
    const int64_t cap = (int64_t) sm_count() * 16;
    if (blocks > cap) blocks = cap;
    return launch(pack_kernel, dim3((unsigned) blocks), dim3(threads), 0, (cudaStream_t) s, dtype, P, first, count,
                  block_bytes(dtype), (const uint8_t *) natural, (uint8_t *) packed, to_packed);
}

int sm100_pack_device(sm100_stream_t s, int dtype, int64_t k, int64_t n, const void * natural, void * packed) {
    return pack_device(s, dtype, k, n, 0, n * (k / (block_elems(dtype) > 0 ? block_elems(dtype) : 1)), natural, packed, 1);
}

int sm100_unpack_device(sm100_stream_t s, int dtype, int64_t k, int64_t n, const void * packed, void * natural) {
    return pack_device(s, dtype, k, n, 0, n * (k / (block_elems(dtype) > 0 ? block_elems(dtype) : 1)), natural, const_cast<void *>(packed), 0);
}

int sm100_pack_device_range(sm100_stream_t s, int dtype, int64_t k, int64_t n, int64_t first_block, int64_t block_count, void * natural_chunk,
                            void * packed, int to_packed) {
    return pack_device(s, dtype, k, n, first_block, block_count, natural_chunk, packed, to_packed);
}

}  // extern "C"
