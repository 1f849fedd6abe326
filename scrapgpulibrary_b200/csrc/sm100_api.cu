// C entry points of the MUL_MAT family: shape checks and the choice between the decode matvec
// (M <= 8, HBM-bound) and the prefill GEMM (tensor cores).
#include "sm100_common.cuh"

#include <cstdlib>

namespace sm100 {
int matvec(cudaStream_t s, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x,
           int64_t ldx, int64_t m, float * y, int64_t ldy);
int matvec_q4k_imma_multi(cudaStream_t s, int count, const void * const * ws, const int64_t * ns, int64_t k, const float * x, int64_t ldx,
                          int64_t m, float * const * ys, const int64_t * ldys, bool * handled, const Q4KPrologue * pro, float * glu_out);
const char * matvec_last_kernel();
void matvec_note_kernel(const char * name);
int matvec_q4k_ring_multi(cudaStream_t s, int count, const void * const * ws, const int64_t * ns, int64_t k, const float * x,
                          float * const * ys, bool * handled, const Q4KPrologue * pro, const ArFuse * fuse);
int gemm_tc_mul_mat(cudaStream_t s, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x,
                    int64_t ldx, int64_t m, float * y, int64_t ldy, bool * handled);
}

using namespace sm100;

extern "C" {

const char * sm100_matvec_last_kernel(void) { return matvec_last_kernel(); }

int sm100_mul_mat(sm100_stream_t s, int dtype, int layout, const void * w, int64_t w_row_stride, int64_t k, int64_t n, const float * x,
                  int64_t ldx, int64_t m, float * y, int64_t ldy) {
    if (m <= 0) return fail(ST_INVALID, "mul_mat: M must be positive");
    if (m <= 8) return matvec((cudaStream_t) s, dtype, layout, w, w_row_stride, k, n, x, ldx, m, y, ldy);
    static const int min_m = [] { const char * e = getenv("SM100_GEMM_MIN_M"); return e != nullptr ? atoi(e) : 33; }();
    if (m >= min_m) {
        if (w == nullptr || x == nullptr || y == nullptr) return fail(ST_INVALID, "mul_mat: null tensor pointer");
        if (k <= 0 || n <= 0) return fail(ST_INVALID, "mul_mat: K, N and M must be positive");
        bool handled = false;
        const int st = gemm_tc_mul_mat((cudaStream_t) s, dtype, layout, w, w_row_stride, k, n, x, ldx, m, y, ldy, &handled);
        if (st != ST_OK || handled) return st;
    }
    // narrow batches, and shapes or dtypes the tensor-core path leaves alone: column panels of 8 through the matvec
    for (int64_t c = 0; c < m; c += 8) {
        const int64_t mm = m - c < 8 ? m - c : 8;
        const int st = matvec((cudaStream_t) s, dtype, layout, w, w_row_stride, k, n, x + c * ldx, ldx, mm, y + c * ldy, ldy);
        if (st != ST_OK) return st;
    }
    return ST_OK;
}

int sm100_mul_mat_multi(sm100_stream_t s, int count, const int * dtypes, const int * layouts, const void * const * ws, int64_t k,
                        const int64_t * ns, const float * x, float * const * ys) {
    if (count < 1 || count > 3 || dtypes == nullptr || layouts == nullptr || ws == nullptr || ns == nullptr || ys == nullptr)
        return fail(ST_INVALID, "mul_mat_multi: 1..3 weight tensors with their dtypes, layouts and outputs are required");
    // packed Q4_K tensors of whole 16-row tiles go out together in one launch; everything else one by one
    const void * gw[3];
    int64_t gn[3], gld[3];
    float * gy[3];
    int grouped = 0;
    bool in_group[3] = {false, false, false};
    for (int i = 0; i < count; ++i) {
        if (ws[i] == nullptr || ys[i] == nullptr || ns[i] <= 0) return fail(ST_INVALID, "mul_mat_multi: null tensor or empty shape");
        if (dtypes[i] == DT_Q4_K && layouts[i] == LAYOUT_PACKED && ns[i] % 16 == 0) {
            gw[grouped] = ws[i]; gn[grouped] = ns[i]; gy[grouped] = ys[i]; gld[grouped] = ns[i];
            in_group[i] = true;
            ++grouped;
        }
    }
    if (grouped >= 2 && x != nullptr && k > 0) {
        bool handled = false;
        int st = matvec_q4k_ring_multi((cudaStream_t) s, grouped, gw, gn, k, x, gy, &handled, nullptr, nullptr);
        if (st != ST_OK) return st;
        if (!handled) st = matvec_q4k_imma_multi((cudaStream_t) s, grouped, gw, gn, k, x, k, 1, gy, gld, &handled, nullptr, nullptr);
        if (st != ST_OK) return st;
        if (!handled) in_group[0] = in_group[1] = in_group[2] = false;
    } else {
        in_group[0] = in_group[1] = in_group[2] = false;
    }
    for (int i = 0; i < count; ++i) {
        if (in_group[i]) continue;
        const int st = matvec((cudaStream_t) s, dtypes[i], layouts[i], ws[i], 0, k, ns[i], x, k, 1, ys[i], ns[i]);
        if (st != ST_OK) return st;
    }
    return ST_OK;
}

int sm100_mul_mat_fused(sm100_stream_t s, int prologue, const float * a, const float * b, const float * norm_w, float eps, float * sum_out,
                        float * x_out, int count, const int * dtypes, const int * layouts, const void * const * ws, int64_t k, const int64_t * ns,
                        float * const * ys) {
    if (count < 1 || count > 3 || dtypes == nullptr || layouts == nullptr || ws == nullptr || ns == nullptr || ys == nullptr || a == nullptr)
        return fail(ST_INVALID, "mul_mat_fused: 1..3 weight tensors with their dtypes, layouts and outputs, and the prologue input, are required");
    if (prologue != SM100_PROLOGUE_SWIGLU && prologue != SM100_PROLOGUE_RMS_NORM) return fail(ST_INVALID, "mul_mat_fused: unknown prologue %d", prologue);
    if (k <= 0) return fail(ST_INVALID, "mul_mat_fused: K must be positive");
    int64_t ld[3];
    for (int i = 0; i < count; ++i) {
        if (ws[i] == nullptr || ys[i] == nullptr || ns[i] <= 0) return fail(ST_INVALID, "mul_mat_fused: null tensor or empty shape");
        if (dtypes[i] != DT_Q4_K || layouts[i] != LAYOUT_PACKED || ns[i] % 16 != 0)
            return fail(ST_UNSUPPORTED, "mul_mat_fused: every weight tensor must be packed Q4_K with a multiple of 16 rows; run the separate ops");
        ld[i] = ns[i];
    }
    if ((sum_out != nullptr && (sum_out == a || sum_out == b)) || (x_out != nullptr && (x_out == a || x_out == b)))
        return fail(ST_INVALID, "mul_mat_fused: sum_out and x_out must not alias the inputs (every CTA reads them while CTA 0 writes)");
    Q4KPrologue pro = {};
    pro.mode = prologue;
    pro.a = a; pro.b = b; pro.norm_w = norm_w; pro.sum_out = sum_out; pro.x_out = x_out; pro.eps = eps;
    bool handled = false;
    int st = matvec_q4k_ring_multi((cudaStream_t) s, count, ws, ns, k, a, ys, &handled, &pro, nullptr);
    if (st != ST_OK) return st;
    if (!handled) st = matvec_q4k_imma_multi((cudaStream_t) s, count, ws, ns, k, a, k, 1, ys, ld, &handled, &pro, nullptr);
    if (st != ST_OK) return st;
    if (!handled) return fail(ST_UNSUPPORTED, "mul_mat_fused: this shape is not served by the fused kernel; run the separate ops");
    return ST_OK;
}

int sm100_mul_mat_glu(sm100_stream_t s, int prologue, const float * a, const float * b, const float * norm_w, float eps, float * sum_out, float * x_out,
                      int dtype, int layout, const void * w_gate, const void * w_up, int64_t k, int64_t n, float * gate_out, float * up_out, float * act_out) {
    if (a == nullptr || w_gate == nullptr || w_up == nullptr || act_out == nullptr || k <= 0 || n <= 0) return fail(ST_INVALID, "mul_mat_glu: null pointer or empty shape");
    if (prologue != 0 && prologue != SM100_PROLOGUE_RMS_NORM) return fail(ST_INVALID, "mul_mat_glu: the prologue is 0 or SM100_PROLOGUE_RMS_NORM");
    if (dtype != DT_Q4_K || layout != LAYOUT_PACKED || n % 16 != 0)
        return fail(ST_UNSUPPORTED, "mul_mat_glu: served for packed Q4_K tensors with a multiple of 16 rows; run the separate ops");
    if ((sum_out != nullptr && (sum_out == a || sum_out == b)) || (x_out != nullptr && (x_out == a || x_out == b)) || act_out == a || act_out == b)
        return fail(ST_INVALID, "mul_mat_glu: the outputs must not alias the inputs (every CTA reads them while others write)");
    Q4KPrologue pro = {};
    pro.mode = prologue;
    pro.a = a; pro.b = b; pro.norm_w = norm_w; pro.sum_out = sum_out; pro.x_out = x_out; pro.eps = eps;
    const void * ws[2] = {w_gate, w_up};
    const int64_t ns[2] = {n, n}, ld[2] = {n, n};
    float * ys[2] = {gate_out, up_out};
    bool handled = false;
    const int st = matvec_q4k_imma_multi((cudaStream_t) s, 2, ws, ns, k, a, k, 1, ys, ld, &handled, prologue != 0 ? &pro : nullptr, act_out);
    if (st != ST_OK) return st;
    if (!handled) return fail(ST_UNSUPPORTED, "mul_mat_glu: this shape is not served by the fused kernel; run the separate ops");
    return ST_OK;
}

int sm100_mul_mat_allreduce(sm100_allreduce_t ctx, sm100_stream_t s, int prologue, const float * a, const float * b, int dtype, int layout,
                            const void * w, int64_t k, int64_t n, float * y) {
    if (ctx == nullptr || a == nullptr || w == nullptr || y == nullptr || k <= 0 || n <= 0) return fail(ST_INVALID, "mul_mat_allreduce: null pointer or empty shape");
    if (prologue != 0 && prologue != SM100_PROLOGUE_SWIGLU) return fail(ST_INVALID, "mul_mat_allreduce: the prologue is 0 or SM100_PROLOGUE_SWIGLU");
    if (prologue == SM100_PROLOGUE_SWIGLU && b == nullptr) return fail(ST_INVALID, "mul_mat_allreduce: SwiGLU needs both halves");
    ArFuse fuse;
    allreduce_fuse_args(ctx, &fuse);
    if (n % 4 != 0 || n > fuse.capacity) return fail(ST_INVALID, "mul_mat_allreduce: N must be a multiple of 4 within the context's capacity");
    if (dtype == DT_Q4_K && layout == LAYOUT_PACKED && fuse.world > 1) {
        Q4KPrologue pro = {};
        pro.mode = prologue;
        pro.a = a; pro.b = b;
        bool handled = false;
        const int st = matvec_q4k_ring_multi((cudaStream_t) s, 1, &w, &n, k, a, &y, &handled, prologue != 0 ? &pro : nullptr, &fuse);
        if (st != ST_OK) return st;
        if (handled) {
            matvec_note_kernel("matvec_q4k_ring+allreduce");
            return ST_OK;
        }
    }
    // the separate launches: (SwiGLU into library scratch,) the matvec, the one-shot all-reduce
    int st;
    if (prologue == SM100_PROLOGUE_SWIGLU) {
        if (dtype == DT_Q4_K && layout == LAYOUT_PACKED && n % 16 == 0) {
            const int dt = dtype, lay = layout;
            st = sm100_mul_mat_fused(s, prologue, a, b, nullptr, 0.0f, nullptr, nullptr, 1, &dt, &lay, &w, k, &n, &y);
        } else {
            return fail(ST_UNSUPPORTED, "mul_mat_allreduce: the SwiGLU prologue is served for packed Q4_K tensors with a multiple of 16 rows; run the separate ops");
        }
    } else {
        st = matvec((cudaStream_t) s, dtype, layout, w, 0, k, n, a, k, 1, y, n);
    }
    if (st != ST_OK) return st;
    return fuse.world > 1 ? sm100_allreduce_sum(ctx, s, y, (int) n) : ST_OK;
}

}  // extern "C"
