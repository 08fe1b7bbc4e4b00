// Row-wise kernels for layers whose norm stands BEHIND the sublayer and whose sublayers read the residual stream itself:
//   x += LN(s) * w, s = a                                             (one sublayer result)
//   x += LN(s) * w, s = (RMS(a) * wa + RMS(b) * wb) / 2               (two results side by side, each RMS-normed first)
// with the stream's rows also handed on in the activation dtype (what the next sublayer's products read), the plain cast
// of rows, and the soft cap c * tanh(x / c) on logits. Statistics and sums are 32-bit; one warp per row, a lane adds in
// index order, the warp's sum is a fixed butterfly: a row's result depends on the row alone.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int ROWS_PER_BLOCK = 4;

template <typename TY>
__global__ void __launch_bounds__(32 * ROWS_PER_BLOCK)
post_norm_residual_kernel(float* x, const float* a, const void* __restrict__ wa, int wa_dtype, const float* b,
                          const void* __restrict__ wb, int wb_dtype, float rms_eps, const void* __restrict__ w, int w_dtype,
                          float eps, TY* __restrict__ y, int rows, int d) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* ar = a + (size_t)r * d;
    const float* br = b ? b + (size_t)r * d : nullptr;
    float inv_a = 1.f, inv_b = 1.f;
    if (br) {
        float sa = 0.f, sb = 0.f;
        for (int i = lane; i < d; i += 32) { sa += ar[i] * ar[i]; sb += br[i] * br[i]; }
        inv_a = 1.0f / sqrtf(bl_warp_sum(sa) / (float)d + rms_eps);
        inv_b = 1.0f / sqrtf(bl_warp_sum(sb) / (float)d + rms_eps);
    }
    auto sub = [&](int i) {
        return br ? 0.5f * (ar[i] * inv_a * bl_load_any(wa, wa_dtype, i) + br[i] * inv_b * bl_load_any(wb, wb_dtype, i)) : ar[i];
    };
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s += sub(i);
    const float mean = bl_warp_sum(s) / (float)d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { const float c = sub(i) - mean; ss += c * c; }
    const float inv = 1.0f / sqrtf(bl_warp_sum(ss) / (float)d + eps);
    float* dst = x + (size_t)r * d;
    for (int i = lane; i < d; i += 32) {
        const float v = dst[i] + (sub(i) - mean) * inv * bl_load_any(w, w_dtype, i);
        dst[i] = v;
        if (y) bl_store(y + (size_t)r * d + i, v);
    }
}

// The same with a block of 128 threads per row and the row in registers (widths up to ROW_MAX): every operand is read
// once, and a short row (a decode step's) does not wait for one warp's chain of loads.
constexpr int ROW_THREADS = 128, ROW_VALS = 32, ROW_MAX = ROW_THREADS * ROW_VALS;
constexpr int ROW_KERNEL_MAX_ROWS = 256;               // with more rows a warp per row fills the device as well (measured: 2,048 rows of 896, 25 us against 40)

__device__ __forceinline__ float row_sum(float v, float* part) {
    v = bl_warp_sum(v);
    __syncthreads();                                   // part may still be read from the call before
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    return (part[0] + part[1]) + (part[2] + part[3]);
}

template <typename TY>
__global__ void __launch_bounds__(ROW_THREADS)
post_norm_residual_row_kernel(float* x, const float* a, const void* __restrict__ wa, int wa_dtype, const float* b,
                              const void* __restrict__ wb, int wb_dtype, float rms_eps, const void* __restrict__ w, int w_dtype,
                              float eps, TY* __restrict__ y, int d) {
    bl_pdl_trigger();
    __shared__ float part[4];
    const int r = blockIdx.x;
    float wv[ROW_VALS], sv[ROW_VALS];
#pragma unroll
    for (int j = 0; j < ROW_VALS; ++j) {                // the norms' weights do not depend on the kernel before
        const int i = threadIdx.x + ROW_THREADS * j;
        wv[j] = i < d ? bl_load_any(w, w_dtype, i) : 0.f;
    }
    bl_pdl_wait();
    if (b) {
        float bv[ROW_VALS], sa = 0.f, sb = 0.f;
#pragma unroll
        for (int j = 0; j < ROW_VALS; ++j) {
            const int i = threadIdx.x + ROW_THREADS * j;
            sv[j] = i < d ? a[(size_t)r * d + i] : 0.f;
            bv[j] = i < d ? b[(size_t)r * d + i] : 0.f;
            sa += sv[j] * sv[j]; sb += bv[j] * bv[j];
        }
        const float inv_a = 1.0f / sqrtf(row_sum(sa, part) / (float)d + rms_eps);
        const float inv_b = 1.0f / sqrtf(row_sum(sb, part) / (float)d + rms_eps);
#pragma unroll
        for (int j = 0; j < ROW_VALS; ++j) {
            const int i = threadIdx.x + ROW_THREADS * j;
            sv[j] = i < d ? 0.5f * (sv[j] * inv_a * bl_load_any(wa, wa_dtype, i) + bv[j] * inv_b * bl_load_any(wb, wb_dtype, i)) : 0.f;
        }
    } else {
#pragma unroll
        for (int j = 0; j < ROW_VALS; ++j) {
            const int i = threadIdx.x + ROW_THREADS * j;
            sv[j] = i < d ? a[(size_t)r * d + i] : 0.f;
        }
    }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_VALS; ++j) s += sv[j];
    const float mean = row_sum(s, part) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_VALS; ++j) {
        const int i = threadIdx.x + ROW_THREADS * j;
        const float c = i < d ? sv[j] - mean : 0.f;
        ss += c * c;
    }
    const float inv = 1.0f / sqrtf(row_sum(ss, part) / (float)d + eps);
#pragma unroll
    for (int j = 0; j < ROW_VALS; ++j) {
        const int i = threadIdx.x + ROW_THREADS * j;
        if (i < d) {
            const float v = x[(size_t)r * d + i] + (sv[j] - mean) * inv * wv[j];
            x[(size_t)r * d + i] = v;
            if (y) bl_store(y + (size_t)r * d + i, v);
        }
    }
}

__global__ void __launch_bounds__(32 * ROWS_PER_BLOCK)
pair_rms_mean_kernel(const float* a, const void* __restrict__ wa, int wa_dtype, const float* b, const void* __restrict__ wb, int wb_dtype,
                     float rms_eps, float* out, int rows, int d) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* ar = a + (size_t)r * d;
    const float* br = b + (size_t)r * d;
    float sa = 0.f, sb = 0.f;
    for (int i = lane; i < d; i += 32) { sa += ar[i] * ar[i]; sb += br[i] * br[i]; }
    const float inv_a = 1.0f / sqrtf(bl_warp_sum(sa) / (float)d + rms_eps), inv_b = 1.0f / sqrtf(bl_warp_sum(sb) / (float)d + rms_eps);
    for (int i = lane; i < d; i += 32)
        out[(size_t)r * d + i] = 0.5f * (ar[i] * inv_a * bl_load_any(wa, wa_dtype, i) + br[i] * inv_b * bl_load_any(wb, wb_dtype, i));
}

// x += ca * a + cb * b, element by element (32-bit): two sublayer results that join the stream with a constant factor each.
__global__ void add_scaled_pair_kernel(float* x, const float* a, float ca, const float* b, float cb, size_t count) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x)
        x[e] += fmaf(ca, a[e], cb * b[e]);
}

// x[r, :] += sigmoid(g[r * ld_g]) * a[r, :]: a sublayer result behind a gate of ONE number per row.
__global__ void add_row_gated_kernel(float* x, const float* a, const float* g, size_t ld_g, int d, size_t count) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x)
        x[e] = fmaf(1.0f / (1.0f + expf(-g[(e / d) * ld_g])), a[e], x[e]);
}

template <typename TY>
__global__ void cast_rows_kernel(const float* x, TY* y, size_t count) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) bl_store(y + e, x[e]);
}

__global__ void softcap_kernel(float* x, size_t count, float cap, float inv_cap) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x)
        x[e] = cap * tanhf(x[e] * inv_cap);
}

}  // namespace

extern "C" int bl_post_norm_residual(float* x, const float* a, const void* wa, int wa_dtype, const float* b, const void* wb,
                                     int wb_dtype, float rms_eps, const void* w, int w_dtype, float eps, void* y, int y_dtype,
                                     int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0 || a == nullptr || w == nullptr || (b != nullptr && (wa == nullptr || wb == nullptr)))
        BL_FAIL("bl_post_norm_residual: bad arguments (d=%d)", d);
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= ROW_MAX && rows <= ROW_KERNEL_MAX_ROWS) {
        if (y == nullptr || y_dtype == BL_F32)
            BL_CUDA(bl_launch_dependent(post_norm_residual_row_kernel<float>, dim3(rows), dim3(ROW_THREADS), 0, s, x, a, wa, wa_dtype, b, wb,
                                        wb_dtype, rms_eps, w, w_dtype, eps, (float*)y, d));
        else if (y_dtype == BL_BF16)
            BL_CUDA(bl_launch_dependent(post_norm_residual_row_kernel<__nv_bfloat16>, dim3(rows), dim3(ROW_THREADS), 0, s, x, a, wa, wa_dtype, b,
                                        wb, wb_dtype, rms_eps, w, w_dtype, eps, (__nv_bfloat16*)y, d));
        else
            BL_FAIL("bl_post_norm_residual: unknown output dtype %d", y_dtype);
        BL_CHECK_LAUNCH("bl_post_norm_residual");
        return 0;
    }
    const dim3 grid((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK), block(32 * ROWS_PER_BLOCK);
    if (y == nullptr || y_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(post_norm_residual_kernel<float>, grid, block, 0, s, x, a, wa, wa_dtype, b, wb, wb_dtype, rms_eps, w,
                                    w_dtype, eps, (float*)y, rows, d));
    else if (y_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(post_norm_residual_kernel<__nv_bfloat16>, grid, block, 0, s, x, a, wa, wa_dtype, b, wb, wb_dtype, rms_eps,
                                    w, w_dtype, eps, (__nv_bfloat16*)y, rows, d));
    else
        BL_FAIL("bl_post_norm_residual: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_post_norm_residual");
    return 0;
}

extern "C" int bl_pair_rms_mean(const float* a, const void* wa, int wa_dtype, const float* b, const void* wb, int wb_dtype, float rms_eps,
                                float* out, int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0 || !a || !b || !wa || !wb) BL_FAIL("bl_pair_rms_mean: bad arguments (d=%d)", d);
    BL_CUDA(bl_launch_dependent(pair_rms_mean_kernel, dim3((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK), dim3(32 * ROWS_PER_BLOCK), 0,
                                (cudaStream_t)stream, a, wa, wa_dtype, b, wb, wb_dtype, rms_eps, out, rows, d));
    BL_CHECK_LAUNCH("bl_pair_rms_mean");
    return 0;
}

extern "C" int bl_cast_rows(const float* x, void* y, int y_dtype, long long count, void* stream) {
    if (count <= 0) return 0;
    const int blocks = (int)((count + 1023) / 1024 < 2048 ? (count + 1023) / 1024 : 2048);
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype == BL_BF16) BL_CUDA(bl_launch_dependent(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, x, (__nv_bfloat16*)y, (size_t)count));
    else if (y_dtype == BL_F32) BL_CUDA(bl_launch_dependent(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, s, x, (float*)y, (size_t)count));
    else BL_FAIL("bl_cast_rows: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_cast_rows");
    return 0;
}

extern "C" int bl_softcap(float* x, long long count, float cap, void* stream) {
    if (count <= 0) return 0;
    if (!(cap > 0.f)) BL_FAIL("bl_softcap: the cap must be positive, got %g", cap);
    const int blocks = (int)((count + 1023) / 1024 < 2048 ? (count + 1023) / 1024 : 2048);
    BL_CUDA(bl_launch_dependent(softcap_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, (size_t)count, cap, 1.0f / cap));
    BL_CHECK_LAUNCH("bl_softcap");
    return 0;
}

extern "C" int bl_add_scaled_pair(float* x, const float* a, float ca, const float* b, float cb, long long count, void* stream) {
    if (count <= 0) return 0;
    if (!x || !a || !b) BL_FAIL("bl_add_scaled_pair: a null operand");
    const int blocks = (int)((count + 1023) / 1024 < 2048 ? (count + 1023) / 1024 : 2048);
    BL_CUDA(bl_launch_dependent(add_scaled_pair_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, a, ca, b, cb, (size_t)count));
    BL_CHECK_LAUNCH("bl_add_scaled_pair");
    return 0;
}

extern "C" int bl_add_row_gated(float* x, const float* a, const float* gate, long long ld_gate, int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    if (!x || !a || !gate || d <= 0 || ld_gate < 1) BL_FAIL("bl_add_row_gated: bad arguments (d=%d)", d);
    const long long count = (long long)rows * d;
    const int blocks = (int)((count + 1023) / 1024 < 2048 ? (count + 1023) / 1024 : 2048);
    BL_CUDA(bl_launch_dependent(add_row_gated_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, a, gate, (size_t)ld_gate, d,
                                (size_t)count));
    BL_CHECK_LAUNCH("bl_add_row_gated");
    return 0;
}
