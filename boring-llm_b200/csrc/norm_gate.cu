// Layer norm with weight and bias, the gated residual with a norm behind the sublayer, the weighted average of the
// residual streams of all layers so far, and element-wise activations. Statistics, gates and sums are 32-bit in
// every engine dtype; a row's result depends only on the row (one warp per row, a lane adds in index order, the
// warp's sum is a fixed butterfly), never on how many rows the call has.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int ROWS_PER_BLOCK = 4;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// y[r, :] = (x[src, :] - mean) / sqrt(var + eps) * w + b, var = mean of the squared deviations.
template <typename TY>
__global__ void __launch_bounds__(32 * ROWS_PER_BLOCK)
layernorm_kernel(const float* x, const int* __restrict__ row_idx, const void* __restrict__ w, int w_dtype,
                 const void* __restrict__ b, int b_dtype, TY* __restrict__ y, int rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* src = x + (size_t)(row_idx ? row_idx[r] : r) * d;
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s += src[i];
    const float mean = bl_warp_sum(s) / (float)d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { const float c = src[i] - mean; ss += c * c; }
    const float inv = 1.0f / sqrtf(bl_warp_sum(ss) / (float)d + eps);
    TY* dst = y + (size_t)r * d;
    for (int i = lane; i < d; i += 32)
        bl_store(dst + i, (src[i] - mean) * inv * bl_load_any(w, w_dtype, i) + (b ? bl_load_any(b, b_dtype, i) : 0.f));
}

// x[r, :] += LN(sub[r, :] * sigmoid(gate[r, :])) * w + b: the gate on a sublayer's result, the norm behind the
// sublayer and the residual sum in one pass. gate may be null (no gate) and has its own row stride.
__global__ void __launch_bounds__(32 * ROWS_PER_BLOCK)
gated_norm_residual_kernel(float* x, const float* sub, const float* gate, int ld_gate, const void* __restrict__ gb, int gb_dtype,
                           const void* __restrict__ w, int w_dtype, const void* __restrict__ b, int b_dtype, int rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* s_row = sub + (size_t)r * d;
    const float* g_row = gate ? gate + (size_t)r * ld_gate : nullptr;
    auto gated = [&](int i) { return g_row ? s_row[i] * sigmoidf_(g_row[i] + (gb ? bl_load_any(gb, gb_dtype, i) : 0.f)) : s_row[i]; };
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s += gated(i);
    const float mean = bl_warp_sum(s) / (float)d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { const float c = gated(i) - mean; ss += c * c; }
    const float inv = 1.0f / sqrtf(bl_warp_sum(ss) / (float)d + eps);
    float* dst = x + (size_t)r * d;
    for (int i = lane; i < d; i += 32)
        dst[i] += (gated(i) - mean) * inv * bl_load_any(w, w_dtype, i) + (b ? bl_load_any(b, b_dtype, i) : 0.f);
}

// out[e] = sum_j c[j] * streams[j * stride + e], j ascending.
__global__ void depth_mix_kernel(const float* streams, size_t stride, const void* __restrict__ c, int c_dtype, int n,
                                 float* out, size_t count) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc = fmaf(bl_load_any(c, c_dtype, j), streams[(size_t)j * stride + e], acc);
        out[e] = acc;
    }
}


// ---- one block per row, the row in registers (widths that are a multiple of 4, up to ROW_THREADS * 4 * ROW_VECS) ----------
constexpr int ROW_THREADS = 128, ROW_VECS = 8;
constexpr int CHAIN_MAX_STREAMS = 512;               // streams the fused average takes (a model of more layers runs the kernels one by one)

__device__ __forceinline__ float row_block_sum(float v, float* part) {
    v = bl_warp_sum(v);
    __syncthreads();                                   // part may still be read from the sum before
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    return (part[0] + part[1]) + (part[2] + part[3]);
}

__device__ __forceinline__ float4 load4_any(const void* p, int dtype, int i) {
    if (dtype == BL_F32) return *reinterpret_cast<const float4*>((const float*)p + i);
    const uint2 u = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// MODE 0: y = LN(x[src]) * w + b (y in TY); MODE 1: x += LN(sub * sigmoid(gate)) * w + b (x 32-bit, in place).
template <typename TY, int MODE>
__global__ void __launch_bounds__(ROW_THREADS)
norm_rows_kernel(const float* in, const int* __restrict__ row_idx, const float* gate, int ld_gate, const void* __restrict__ gb,
                 int gb_dtype, const void* __restrict__ w, int w_dtype, const void* __restrict__ b, int b_dtype, TY* y, float* x,
                 int d, float eps) {
    bl_pdl_trigger();
    bl_pdl_wait();
    __shared__ float part[4];
    const int r = blockIdx.x, n4 = d >> 2;
    const float4* src = reinterpret_cast<const float4*>(in + (size_t)(row_idx ? row_idx[r] : r) * d);
    const float4* g4 = gate ? reinterpret_cast<const float4*>(gate + (size_t)r * ld_gate) : nullptr;
    float4 v[ROW_VECS];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_VECS; ++j) {
        const int i = threadIdx.x + j * ROW_THREADS;
        if (i < n4) {
            float4 a = src[i];
            if (MODE == 1 && g4) {
                float4 g = g4[i];
                if (gb) { const float4 t = load4_any(gb, gb_dtype, 4 * i); g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w; }
                a.x *= sigmoidf_(g.x); a.y *= sigmoidf_(g.y); a.z *= sigmoidf_(g.z); a.w *= sigmoidf_(g.w);
            }
            v[j] = a;
            s += (a.x + a.y) + (a.z + a.w);
        }
    }
    const float mean = row_block_sum(s, part) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_VECS; ++j) {
        const int i = threadIdx.x + j * ROW_THREADS;
        if (i < n4) {
            const float c0 = v[j].x - mean, c1 = v[j].y - mean, c2 = v[j].z - mean, c3 = v[j].w - mean;
            ss += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
        }
    }
    const float inv = 1.0f / sqrtf(row_block_sum(ss, part) / (float)d + eps);
#pragma unroll
    for (int j = 0; j < ROW_VECS; ++j) {
        const int i = threadIdx.x + j * ROW_THREADS;
        if (i < n4) {
            const float4 ww = load4_any(w, w_dtype, 4 * i);
            const float4 bb = b ? load4_any(b, b_dtype, 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float o0 = (v[j].x - mean) * inv * ww.x + bb.x, o1 = (v[j].y - mean) * inv * ww.y + bb.y;
            const float o2 = (v[j].z - mean) * inv * ww.z + bb.z, o3 = (v[j].w - mean) * inv * ww.w + bb.w;
            if (MODE == 1) {
                float4* dst = reinterpret_cast<float4*>(x + (size_t)r * d) + i;
                float4 cur = *dst;
                cur.x += o0; cur.y += o1; cur.z += o2; cur.w += o3;
                *dst = cur;
            } else if (sizeof(TY) == 4) {
                reinterpret_cast<float4*>(y + (size_t)r * d)[i] = make_float4(o0, o1, o2, o3);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                reinterpret_cast<uint2*>(y + (size_t)r * d)[i] = pk;
            }
        }
    }
}

bool rows_fast(int d, const void* a, const void* b2, const void* c, const void* w, const void* bias, int ld_gate) {
    return d % 4 == 0 && d <= ROW_THREADS * 4 * ROW_VECS && ld_gate % 4 == 0 &&
           (((uintptr_t)a | (uintptr_t)b2 | (uintptr_t)c | (uintptr_t)w | (uintptr_t)bias) & 15) == 0;
}


// Up to three row-wise steps on one row held in registers, each optional, in the order a layer's end needs them:
//   A  x += LN(sub * sigmoid(gate + gate_bias)) * w + b            (sub null: the row is x as it stands)
//   B  mixed = sum_{j < n - 1} c[j] * streams[j] + c[n - 1] * row   (the row is stream n - 1); written to mix_out
//   C  y = LN(row) * w2 + b2                                         (the norm that reads the row next)
// Every step does what its own kernel does, in the same order of operations: fusing changes no bit.
template <typename TY>
__global__ void __launch_bounds__(ROW_THREADS)
norm_chain_kernel(float* x, const float* sub, const float* gate, int ld_gate, const void* __restrict__ gb, int gb_dtype,
                  const void* __restrict__ w, int w_dtype, const void* __restrict__ b, int b_dtype, float eps,
                  const float* streams, size_t stride, const void* __restrict__ c, int c_dtype, int n, float* mix_out,
                  const void* __restrict__ w2, int w2_dtype, const void* __restrict__ b2, int b2_dtype, float eps2, TY* y, int d) {
    bl_pdl_trigger();
    __shared__ float part[4];
    __shared__ float cw[CHAIN_MAX_STREAMS];            // the average's weights: model constants, fetched before the wait
    if (streams)
        for (int k = threadIdx.x; k < n; k += ROW_THREADS) cw[k] = bl_load_any(c, c_dtype, k);
    bl_pdl_wait();
    const int r = blockIdx.x, n4 = d >> 2;
    float4 v[ROW_VECS];
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * d);
    if (sub) {
        const float4* src = reinterpret_cast<const float4*>(sub + (size_t)r * d);
        const float4* g4 = gate ? reinterpret_cast<const float4*>(gate + (size_t)r * ld_gate) : nullptr;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) {
                float4 a = src[i];
                if (g4) {
                    float4 g = g4[i];
                    if (gb) { const float4 t = load4_any(gb, gb_dtype, 4 * i); g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w; }
                    a.x *= sigmoidf_(g.x); a.y *= sigmoidf_(g.y); a.z *= sigmoidf_(g.z); a.w *= sigmoidf_(g.w);
                }
                v[j] = a;
                s += (a.x + a.y) + (a.z + a.w);
            }
        }
        const float mean = row_block_sum(s, part) / (float)d;
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) {
                const float c0 = v[j].x - mean, c1 = v[j].y - mean, c2 = v[j].z - mean, c3 = v[j].w - mean;
                ss += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
            }
        }
        const float inv = 1.0f / sqrtf(row_block_sum(ss, part) / (float)d + eps);
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) {
                const float4 ww = load4_any(w, w_dtype, 4 * i);
                const float4 bb = b ? load4_any(b, b_dtype, 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 cur = xr[i];
                cur.x += (v[j].x - mean) * inv * ww.x + bb.x; cur.y += (v[j].y - mean) * inv * ww.y + bb.y;
                cur.z += (v[j].z - mean) * inv * ww.z + bb.z; cur.w += (v[j].w - mean) * inv * ww.w + bb.w;
                xr[i] = cur;
                v[j] = cur;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) v[j] = xr[i];
        }
    }
    if (streams) {
        const float4* st4 = reinterpret_cast<const float4*>(streams) + (size_t)r * n4;
        const size_t stride4 = stride >> 2;
        float4* mo = reinterpret_cast<float4*>(mix_out + (size_t)r * d);
        // stream by stream, a thread's loads of one stream in flight together (the sum of an element stays in ascending j)
        float4 acc[ROW_VECS];
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        __syncthreads();                               // cw is written
#pragma unroll 4
        for (int k = 0; k < n - 1; ++k) {
            const float ck = cw[k];
            const float4* sk4 = st4 + (size_t)k * stride4;
#pragma unroll
            for (int j = 0; j < ROW_VECS; ++j) {
                const int i = threadIdx.x + j * ROW_THREADS;
                if (i < n4) {
                    const float4 a = sk4[i];
                    acc[j].x = fmaf(ck, a.x, acc[j].x); acc[j].y = fmaf(ck, a.y, acc[j].y);
                    acc[j].z = fmaf(ck, a.z, acc[j].z); acc[j].w = fmaf(ck, a.w, acc[j].w);
                }
            }
        }
        const float cl = cw[n - 1];
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) {
                acc[j].x = fmaf(cl, v[j].x, acc[j].x); acc[j].y = fmaf(cl, v[j].y, acc[j].y);
                acc[j].z = fmaf(cl, v[j].z, acc[j].z); acc[j].w = fmaf(cl, v[j].w, acc[j].w);
                mo[i] = acc[j];
                v[j] = acc[j];
            }
        }
    }
    if (w2) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        }
        const float mean = row_block_sum(s, part) / (float)d;
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) {
                const float c0 = v[j].x - mean, c1 = v[j].y - mean, c2 = v[j].z - mean, c3 = v[j].w - mean;
                ss += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
            }
        }
        const float inv = 1.0f / sqrtf(row_block_sum(ss, part) / (float)d + eps2);
#pragma unroll
        for (int j = 0; j < ROW_VECS; ++j) {
            const int i = threadIdx.x + j * ROW_THREADS;
            if (i < n4) {
                const float4 ww = load4_any(w2, w2_dtype, 4 * i);
                const float4 bb = b2 ? load4_any(b2, b2_dtype, 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float o0 = (v[j].x - mean) * inv * ww.x + bb.x, o1 = (v[j].y - mean) * inv * ww.y + bb.y;
                const float o2 = (v[j].z - mean) * inv * ww.z + bb.z, o3 = (v[j].w - mean) * inv * ww.w + bb.w;
                if (sizeof(TY) == 4) {
                    reinterpret_cast<float4*>(y + (size_t)r * d)[i] = make_float4(o0, o1, o2, o3);
                } else {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
                    uint2 pk;
                    pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                    reinterpret_cast<uint2*>(y + (size_t)r * d)[i] = pk;
                }
            }
        }
    }
}

// out[e] = sum_j c[j] * streams[j * stride + e], four values at a time.
__global__ void depth_mix4_kernel(const float4* streams, size_t stride4, const void* __restrict__ c, int c_dtype, int n,
                                  float4* out, size_t count4) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count4; e += (size_t)gridDim.x * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < n; ++j) {
            const float cj = bl_load_any(c, c_dtype, j);
            const float4 a = streams[(size_t)j * stride4 + e];
            acc.x = fmaf(cj, a.x, acc.x); acc.y = fmaf(cj, a.y, acc.y); acc.z = fmaf(cj, a.z, acc.z); acc.w = fmaf(cj, a.w, acc.w);
        }
        out[e] = acc;
    }
}

template <typename TI, typename TO, int ACT>
__global__ void activation_kernel(const TI* x, TO* y, size_t count, int cols, size_t ld_x, size_t ld_y) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / cols, c = e % cols;
        const float v = bl_load(x + r * ld_x + c);
        float o;
        if (ACT == BL_ACT_GELU_ERF) o = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
        else if (ACT == BL_ACT_GELU_TANH) o = 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
        else o = bl_silu(v);
        bl_store(y + r * ld_y + c, o);
    }
}

// Gated activations on the 32-bit sums of a joined product: row r holds `cols` gate sums, then `cols` up sums;
// y[r, c] = bl_glu(kind, gate, up, limit) (common.cuh).
template <typename TO>
__global__ void glu_act_kernel(const float* x, TO* y, size_t count, int cols, size_t ld_x, size_t ld_y, int kind, float limit) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / cols, c = e % cols;
        bl_store(y + r * ld_y + c, bl_glu(kind, x[r * ld_x + c], x[r * ld_x + cols + c], limit));
    }
}

// The gated activations, four hidden units a thread: cols and both row strides multiples of 4, 16-byte aligned rows.
template <typename TO>
__global__ void glu_act4_kernel(const float* x, TO* y, size_t count4, int cols4, size_t ld_x, size_t ld_y, int kind, float limit) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count4; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / cols4, c = (e % cols4) * 4;
        const float4 g = *reinterpret_cast<const float4*>(x + r * ld_x + c);
        const float4 u = *reinterpret_cast<const float4*>(x + r * ld_x + (size_t)cols4 * 4 + c);
        const float o0 = bl_glu(kind, g.x, u.x, limit), o1 = bl_glu(kind, g.y, u.y, limit);
        const float o2 = bl_glu(kind, g.z, u.z, limit), o3 = bl_glu(kind, g.w, u.w, limit);
        TO* dst = y + r * ld_y + c;
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 a = __floats2bfloat162_rn(o0, o1), b = __floats2bfloat162_rn(o2, o3);
            uint2 v;
            v.x = *reinterpret_cast<unsigned*>(&a); v.y = *reinterpret_cast<unsigned*>(&b);
            *reinterpret_cast<uint2*>(dst) = v;
        }
    }
}

// The same, four values a thread: 32-bit rows in, cols and both row strides multiples of 4, 16-byte aligned.
template <typename TO, int ACT>
__global__ void activation4_kernel(const float* x, TO* y, size_t count4, int cols4, size_t ld_x, size_t ld_y) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count4; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / cols4, c = (e % cols4) * 4;
        const float4 a = *reinterpret_cast<const float4*>(x + r * ld_x + c);
        float o[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float v = o[k];
            if (ACT == BL_ACT_GELU_ERF) o[k] = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
            else if (ACT == BL_ACT_GELU_TANH) o[k] = 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
            else o[k] = bl_silu(v);
        }
        if (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(y + r * ld_y + c) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
            *reinterpret_cast<uint2*>(y + r * ld_y + c) = pk;
        }
    }
}

// xIELU with its two numbers made ready (args = {softplus(p), 1/2 + softplus(q)}, 32-bit on the device):
// v > 0: args[0] v^2 + v / 2;  v <= 0: args[1] (e^v - 1 - v) + v / 2. x: 32-bit sums.
template <typename TO>
__global__ void xielu_kernel(const float* x, TO* y, size_t count, int cols, size_t ld_x, size_t ld_y, const float* __restrict__ args) {
    bl_pdl_trigger();
    const float ap = args[0], an = args[1];
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / cols, c = e % cols;
        const float v = x[r * ld_x + c];
        bl_store(y + r * ld_y + c, bl_xielu(v, ap, an));
    }
}

// The same, four values a thread: cols and both row strides multiples of 4, 16-byte aligned rows.
template <typename TO>
__global__ void xielu4_kernel(const float* x, TO* y, size_t count4, int cols4, size_t ld_x, size_t ld_y, const float* __restrict__ args) {
    bl_pdl_trigger();
    const float ap = args[0], an = args[1];
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count4; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / cols4, c = (e % cols4) * 4;
        const float4 a = *reinterpret_cast<const float4*>(x + r * ld_x + c);
        const float o0 = bl_xielu(a.x, ap, an), o1 = bl_xielu(a.y, ap, an), o2 = bl_xielu(a.z, ap, an), o3 = bl_xielu(a.w, ap, an);
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(y + r * ld_y + c) = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            uint2 pk;
            pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
            *reinterpret_cast<uint2*>(y + r * ld_y + c) = pk;
        }
    }
}

int grid_for(size_t count, int threads) {
    size_t b = (count + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

extern "C" int bl_layernorm(const float* x, const int* row_idx, const void* w, int w_dtype, const void* b, int b_dtype,
                            void* y, int y_dtype, int rows, int d, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0) BL_FAIL("bl_layernorm: bad width %d", d);
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype != BL_F32 && y_dtype != BL_BF16) BL_FAIL("bl_layernorm: unknown output dtype %d", y_dtype);
    if (rows_fast(d, x, y, nullptr, w, b, 0)) {
        if (y_dtype == BL_F32)
            BL_CUDA(bl_launch_dependent(norm_rows_kernel<float, 0>, dim3(rows), dim3(ROW_THREADS), 0, s, x, row_idx, nullptr, 0, nullptr, 0, w, w_dtype, b, b_dtype, (float*)y, (float*)nullptr, d, eps));
        else
            BL_CUDA(bl_launch_dependent(norm_rows_kernel<__nv_bfloat16, 0>, dim3(rows), dim3(ROW_THREADS), 0, s, x, row_idx, nullptr, 0, nullptr, 0, w, w_dtype, b, b_dtype,
                                                                             (__nv_bfloat16*)y, (float*)nullptr, d, eps));
        BL_CHECK_LAUNCH("bl_layernorm");
        return 0;
    }
    const int blocks = (rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
    if (y_dtype == BL_F32)
        layernorm_kernel<float><<<blocks, 32 * ROWS_PER_BLOCK, 0, s>>>(x, row_idx, w, w_dtype, b, b_dtype, (float*)y, rows, d, eps);
    else if (y_dtype == BL_BF16)
        layernorm_kernel<__nv_bfloat16><<<blocks, 32 * ROWS_PER_BLOCK, 0, s>>>(x, row_idx, w, w_dtype, b, b_dtype,
                                                                                 (__nv_bfloat16*)y, rows, d, eps);
    else
        BL_FAIL("bl_layernorm: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_layernorm");
    return 0;
}

extern "C" int bl_gated_norm_residual(float* x, const float* sub, const float* gate, int ld_gate, const void* gate_bias,
                                      int gb_dtype, const void* w, int w_dtype, const void* b, int b_dtype, int rows, int d,
                                      float eps, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0 || (gate && ld_gate < d)) BL_FAIL("bl_gated_norm_residual: bad width %d or gate stride %d", d, ld_gate);
    if (rows_fast(d, x, sub, gate, w, b, gate ? ld_gate : 0) && ((uintptr_t)gate_bias & 15) == 0) {
        BL_CUDA(bl_launch_dependent(norm_rows_kernel<float, 1>, dim3(rows), dim3(ROW_THREADS), 0, (cudaStream_t)stream, sub, (const int*)nullptr, gate, ld_gate, gate_bias, gb_dtype, w,
                                                                                   w_dtype, b, b_dtype, (float*)nullptr, x, d, eps));
        BL_CHECK_LAUNCH("bl_gated_norm_residual");
        return 0;
    }
    const int blocks = (rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
    gated_norm_residual_kernel<<<blocks, 32 * ROWS_PER_BLOCK, 0, (cudaStream_t)stream>>>(x, sub, gate, ld_gate, gate_bias, gb_dtype, w,
                                                                                         w_dtype, b, b_dtype, rows, d, eps);
    BL_CHECK_LAUNCH("bl_gated_norm_residual");
    return 0;
}

extern "C" int bl_depth_mix(const float* streams, long long stride, const void* coeffs, int c_dtype, int n, float* out,
                            long long count, void* stream) {
    if (count <= 0) return 0;
    if (n <= 0 || stride < count) BL_FAIL("bl_depth_mix: %d streams with stride %lld for %lld values", n, stride, count);
    if (count % 4 == 0 && stride % 4 == 0 && (((uintptr_t)streams | (uintptr_t)out) & 15) == 0) {
        BL_CUDA(bl_launch_dependent(depth_mix4_kernel, dim3(grid_for((size_t)count / 4, 256)), dim3(256), 0, (cudaStream_t)stream,
                                    (const float4*)streams, (size_t)stride / 4, coeffs, c_dtype, n, (float4*)out, (size_t)count / 4));
        BL_CHECK_LAUNCH("bl_depth_mix");
        return 0;
    }
    depth_mix_kernel<<<grid_for((size_t)count, 256), 256, 0, (cudaStream_t)stream>>>(streams, (size_t)stride, coeffs, c_dtype, n,
                                                                                     out, (size_t)count);
    BL_CHECK_LAUNCH("bl_depth_mix");
    return 0;
}

extern "C" int bl_glu_act(const float* x, long long ld_x, void* y, int y_dtype, long long ld_y, int rows, int cols, int kind,
                          float limit, void* stream) {
    const long long count = (long long)rows * cols;
    if (count <= 0) return 0;
    if (ld_x < 2 * (long long)cols || ld_y < cols) BL_FAIL("bl_glu_act: rows of 2 x %d sums are %lld apart, results %lld", cols, ld_x, ld_y);
    if (kind != BL_GLU_SILU && kind != BL_GLU_GELU_TANH && kind != BL_GLU_CLAMPED) BL_FAIL("bl_glu_act: unknown kind %d", kind);
    cudaStream_t s = (cudaStream_t)stream;
    if (cols % 4 == 0 && ld_x % 4 == 0 && ld_y % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0 && (y_dtype == BL_F32 || y_dtype == BL_BF16)) {
        const long long count4 = count / 4;
        const int g4 = (int)((count4 + 255) / 256 < 148 * 16 ? (count4 + 255) / 256 : 148 * 16);
        if (y_dtype == BL_F32) BL_CUDA(bl_launch_dependent(glu_act4_kernel<float>, dim3(g4), dim3(256), 0, s, x, (float*)y, (size_t)count4, cols / 4, (size_t)ld_x, (size_t)ld_y, kind, limit));
        else BL_CUDA(bl_launch_dependent(glu_act4_kernel<__nv_bfloat16>, dim3(g4), dim3(256), 0, s, x, (__nv_bfloat16*)y, (size_t)count4, cols / 4, (size_t)ld_x, (size_t)ld_y, kind, limit));
        BL_CHECK_LAUNCH("bl_glu_act");
        return 0;
    }
    const int g = (int)((count + 255) / 256 < 148 * 16 ? (count + 255) / 256 : 148 * 16);
    if (y_dtype == BL_F32) BL_CUDA(bl_launch_dependent(glu_act_kernel<float>, dim3(g), dim3(256), 0, s, x, (float*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y, kind, limit));
    else if (y_dtype == BL_BF16) BL_CUDA(bl_launch_dependent(glu_act_kernel<__nv_bfloat16>, dim3(g), dim3(256), 0, s, x, (__nv_bfloat16*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y, kind, limit));
    else BL_FAIL("bl_glu_act: unknown dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_glu_act");
    return 0;
}

extern "C" int bl_activation(const void* x, int x_dtype, long long ld_x, void* y, int y_dtype, long long ld_y, int rows, int cols,
                             int act, void* stream) {
    const long long count = (long long)rows * cols;
    if (count <= 0) return 0;
    if (ld_x < cols || ld_y < cols) BL_FAIL("bl_activation: rows of %d values are %lld and %lld apart", cols, ld_x, ld_y);
    cudaStream_t s = (cudaStream_t)stream;
    const int g = grid_for((size_t)count, 256);
    if (act != BL_ACT_SILU && act != BL_ACT_GELU_ERF && act != BL_ACT_GELU_TANH) BL_FAIL("bl_activation: unknown activation %d", act);
    if (x_dtype == BL_F32 && cols % 4 == 0 && ld_x % 4 == 0 && ld_y % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
        const size_t count4 = (size_t)count / 4;
        const int g4 = grid_for(count4, 256);
#define BL_GO4(TO) do { \
        if (act == BL_ACT_GELU_ERF) BL_CUDA(bl_launch_dependent(activation4_kernel<TO, BL_ACT_GELU_ERF>, dim3(g4), dim3(256), 0, s, (const float*)x, (TO*)y, count4, cols / 4, (size_t)ld_x, (size_t)ld_y)); \
        else if (act == BL_ACT_GELU_TANH) BL_CUDA(bl_launch_dependent(activation4_kernel<TO, BL_ACT_GELU_TANH>, dim3(g4), dim3(256), 0, s, (const float*)x, (TO*)y, count4, cols / 4, (size_t)ld_x, (size_t)ld_y)); \
        else BL_CUDA(bl_launch_dependent(activation4_kernel<TO, BL_ACT_SILU>, dim3(g4), dim3(256), 0, s, (const float*)x, (TO*)y, count4, cols / 4, (size_t)ld_x, (size_t)ld_y)); } while (0)
        if (y_dtype == BL_F32) { BL_GO4(float); BL_CHECK_LAUNCH("bl_activation"); return 0; }
        if (y_dtype == BL_BF16) { BL_GO4(__nv_bfloat16); BL_CHECK_LAUNCH("bl_activation"); return 0; }
#undef BL_GO4
    }
#define BL_GO3(TI, TO) do { \
        if (act == BL_ACT_GELU_ERF) BL_CUDA(bl_launch_dependent(activation_kernel<TI, TO, BL_ACT_GELU_ERF>, dim3(g), dim3(256), 0, s, (const TI*)x, (TO*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y)); \
        else if (act == BL_ACT_GELU_TANH) BL_CUDA(bl_launch_dependent(activation_kernel<TI, TO, BL_ACT_GELU_TANH>, dim3(g), dim3(256), 0, s, (const TI*)x, (TO*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y)); \
        else BL_CUDA(bl_launch_dependent(activation_kernel<TI, TO, BL_ACT_SILU>, dim3(g), dim3(256), 0, s, (const TI*)x, (TO*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y)); } while (0)
    if (x_dtype == BL_F32 && y_dtype == BL_F32) BL_GO3(float, float);
    else if (x_dtype == BL_F32 && y_dtype == BL_BF16) BL_GO3(float, __nv_bfloat16);
    else if (x_dtype == BL_BF16 && y_dtype == BL_BF16) BL_GO3(__nv_bfloat16, __nv_bfloat16);
    else BL_FAIL("bl_activation: unsupported dtypes %d -> %d", x_dtype, y_dtype);
#undef BL_GO3
    BL_CHECK_LAUNCH("bl_activation");
    return 0;
}

extern "C" int bl_norm_chain_supported(int d, int ld_gate) {
    return d > 0 && d % 4 == 0 && d <= ROW_THREADS * 4 * ROW_VECS && ld_gate % 4 == 0;
}

extern "C" int bl_norm_chain(float* x, const float* sub, const float* gate, int ld_gate, const void* gate_bias, int gb_dtype,
                             const void* w, int w_dtype, const void* b, int b_dtype, float eps, const float* streams,
                             long long stride, const void* coeffs, int c_dtype, int n, float* mix_out, const void* w2, int w2_dtype,
                             const void* b2, int b2_dtype, float eps2, void* y, int y_dtype, int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    if (!bl_norm_chain_supported(d, gate ? ld_gate : 0)) BL_FAIL("bl_norm_chain: width %d or gate stride %d is not built", d, ld_gate);
    if ((((uintptr_t)x | (uintptr_t)sub | (uintptr_t)gate | (uintptr_t)gate_bias | (uintptr_t)w | (uintptr_t)b | (uintptr_t)streams |
          (uintptr_t)mix_out | (uintptr_t)w2 | (uintptr_t)b2 | (uintptr_t)y) & 15) != 0 || stride % 4 != 0)
        BL_FAIL("bl_norm_chain: every operand must be 16-byte aligned");
    if (streams && (n < 1 || n > CHAIN_MAX_STREAMS || mix_out == nullptr || coeffs == nullptr))
        BL_FAIL("bl_norm_chain: the average needs 1..%d streams, weights and a place to go", CHAIN_MAX_STREAMS);
    if (w2 && y == nullptr) BL_FAIL("bl_norm_chain: the norm needs a place to go");
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(norm_chain_kernel<__nv_bfloat16>, dim3(rows), dim3(ROW_THREADS), 0, s, x, sub, gate, ld_gate, gate_bias,
                                    gb_dtype, w, w_dtype, b, b_dtype, eps, streams, (size_t)stride, coeffs, c_dtype, n, mix_out, w2, w2_dtype,
                                    b2, b2_dtype, eps2, (__nv_bfloat16*)y, d));
    else if (y_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(norm_chain_kernel<float>, dim3(rows), dim3(ROW_THREADS), 0, s, x, sub, gate, ld_gate, gate_bias,
                                    gb_dtype, w, w_dtype, b, b_dtype, eps, streams, (size_t)stride, coeffs, c_dtype, n, mix_out, w2, w2_dtype,
                                    b2, b2_dtype, eps2, (float*)y, d));
    else
        BL_FAIL("bl_norm_chain: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_norm_chain");
    return 0;
}

extern "C" int bl_xielu(const float* x, long long ld_x, void* y, int y_dtype, long long ld_y, int rows, int cols, const float* args,
                        void* stream) {
    const long long count = (long long)rows * cols;
    if (count <= 0) return 0;
    if (ld_x < cols || ld_y < cols || !args) BL_FAIL("bl_xielu: rows of %d values are %lld and %lld apart", cols, ld_x, ld_y);
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype != BL_F32 && y_dtype != BL_BF16) BL_FAIL("bl_xielu: unknown dtype %d", y_dtype);
    if (cols % 4 == 0 && ld_x % 4 == 0 && ld_y % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & (y_dtype == BL_F32 ? 15 : 7)) == 0) {
        const size_t count4 = (size_t)count / 4;
        const int g4 = grid_for(count4, 256);
        if (y_dtype == BL_F32) BL_CUDA(bl_launch_dependent(xielu4_kernel<float>, dim3(g4), dim3(256), 0, s, x, (float*)y, count4, cols / 4, (size_t)ld_x, (size_t)ld_y, args));
        else BL_CUDA(bl_launch_dependent(xielu4_kernel<__nv_bfloat16>, dim3(g4), dim3(256), 0, s, x, (__nv_bfloat16*)y, count4, cols / 4, (size_t)ld_x, (size_t)ld_y, args));
        BL_CHECK_LAUNCH("bl_xielu");
        return 0;
    }
    const int g = grid_for((size_t)count, 256);
    if (y_dtype == BL_F32) BL_CUDA(bl_launch_dependent(xielu_kernel<float>, dim3(g), dim3(256), 0, s, x, (float*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y, args));
    else if (y_dtype == BL_BF16) BL_CUDA(bl_launch_dependent(xielu_kernel<__nv_bfloat16>, dim3(g), dim3(256), 0, s, x, (__nv_bfloat16*)y, (size_t)count, cols, (size_t)ld_x, (size_t)ld_y, args));
    else BL_FAIL("bl_xielu: unknown dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_xielu");
    return 0;
}
