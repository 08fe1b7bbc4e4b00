// Routed experts: the choice of experts per token, matrix products whose rows each use the matrix of their own expert, and
// the weighted sum of a token's expert results.
//   scores s = sigmoid(z), or softmax(z) over all experts (z: the router's 32-bit logits); choice scores c = s + correction;
//   the experts are n_groups equal runs of neighbours, a group's score is the sum of its two largest choice scores (its only
//   one where groups hold one expert) or its largest alone, only experts of the `keep` best groups can be chosen; the `top`
//   largest choice scores among them are chosen (ties: the lower index); the weights are the chosen experts' s, as they are.
//   Expert numbers from n_real on are identity experts: they have no matrices, no rows in the products, and the weighted sum
//   takes the token's input row in their place.
// Everything here is a function of the token's row alone: a token's experts, weights and sums do not depend on the batch.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// One warp per token. Shared memory: s [E], c [E], group scores [n_groups], kept flags [n_groups].
__global__ void __launch_bounds__(32)
moe_route_kernel(const float* __restrict__ z, int ldz, const void* __restrict__ corr, int corr_dtype, int E, int top, int n_groups,
                 int keep, int* __restrict__ ids, float* __restrict__ wts, int score_kind, int group_top) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ float sm[];
    float* s = sm;
    float* c = sm + E;
    float* gs = sm + 2 * E;
    float* kept = gs + n_groups;
    const int t = blockIdx.x, lane = threadIdx.x;
    const int per = E / n_groups;
    float zmax = -INFINITY, zsum = 1.f;
    if (score_kind == BL_SCORE_SOFTMAX) {                      // the maximum and the denominator, lanes in a fixed order
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[(size_t)t * ldz + e]);
        zmax = bl_warp_max(zmax);
        float part = 0.f;
        for (int e = lane; e < E; e += 32) part += expf(z[(size_t)t * ldz + e] - zmax);
        zsum = bl_warp_sum(part);
    }
    for (int e = lane; e < E; e += 32) {
        const float ze = z[(size_t)t * ldz + e];
        const float v = score_kind == BL_SCORE_SOFTMAX ? expf(ze - zmax) / zsum : 1.0f / (1.0f + expf(-ze));
        s[e] = v;
        c[e] = v + (corr ? bl_load_any(corr, corr_dtype, e) : 0.f);
    }
    __syncwarp();
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;                // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = c[e];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = per > 1 && group_top > 1 ? a + b : a;
            kept[g] = 0.f;
        }
        __syncwarp();
        // the groups that are NOT kept lose their experts: take the best `keep` out, then close the rest
        for (int n = 0; n < keep; ++n) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) if (gs[g] > bv || (gs[g] == bv && g < bi)) { bv = gs[g]; bi = g; }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < n_groups) { gs[bi] = -INFINITY; kept[bi] = 1.f; }
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (kept[e / per] == 0.f) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int n = 0; n < top; ++n) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) if (c[e] > bv || (c[e] == bv && e < bi)) { bv = c[e]; bi = e; }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;                                   // fewer open experts than `top` (refused on the host)
        if (lane == 0) {
            ids[(size_t)t * top + n] = bi;
            wts[(size_t)t * top + n] = s[bi];
            c[bi] = -INFINITY;
        }
        __syncwarp();
    }
}

// Experts chosen by a table over token ids instead of a router: ids[t, :] = table[token[t], :], every weight 1 / top.
__global__ void table_route_kernel(const int* __restrict__ table, const int* __restrict__ tokens, int T, int top, int* __restrict__ ids,
                                   float* __restrict__ wts) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= T * top) return;
    ids[e] = table[(size_t)tokens[e / top] * top + e % top];
    wts[e] = 1.0f / (float)top;
}

// out[p, n] = epilogue(x[p / x_div, :] . W[ids[p]][n, :]), one warp per output (the lanes over k, a fixed butterfly):
// the plain product for rows that each have their own matrix. SWIGLU: W[e] holds N gate rows, then N up rows.
template <typename TX, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(WARPS * 32)
expert_gemm_plain_kernel(const TX* __restrict__ x, int x_div, const TW* __restrict__ w, size_t expert_stride,
                         const int* __restrict__ ids, TO* __restrict__ out, int P, int N, int K, const float* __restrict__ act, int n_real) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * WARPS + (threadIdx.x >> 5);
    const int p = blockIdx.y;
    if (n >= N || ids[p] >= n_real) return;                    // an identity expert has no matrix: its row is never read
    const TX* xr = x + (size_t)(p / x_div) * K;
    const TW* wr = w + (size_t)ids[p] * expert_stride + (size_t)n * K;
    float a = 0.f, u = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float xv = bl_load(xr + k);
        a = fmaf(xv, bl_load(wr + k), a);
        if (EPI == BL_EPI_SWIGLU) u = fmaf(xv, bl_load(wr + (size_t)N * K + k), u);
    }
    a = bl_warp_sum(a);
    if (EPI == BL_EPI_SWIGLU) {
        const BlGluArgs glu = bl_glu_args(act);
        a = bl_glu(glu.kind, a, bl_warp_sum(u), glu.limit);
    }
    if (lane == 0) bl_store(out + (size_t)p * N + n, a);
}

// out[t, :] = (add ? out[t, :] : 0) + sum_k wts[t, k] * y[t * top + k, :], k ascending; a pair whose expert is an identity
// expert (ids given, ids[t * top + k] >= n_real) takes x[t, :] in the place of its row of y.
template <typename TX>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, float* out, int top, int d,
                                   size_t count, int add, const int* __restrict__ ids, int n_real, const TX* __restrict__ x) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / d, c = e % d;
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool same = ids && ids[t * top + k] >= n_real;
            acc = fmaf(wts[t * top + k], same ? bl_load(x + t * d + c) : y[(t * top + k) * d + c], acc);
        }
        out[e] = add ? out[e] + acc : acc;
    }
}

// The rows of a grouped product: pairs (token, chosen expert) laid out expert by expert in tiles of `tile` rows, every
// expert's rows starting a new tile. One block. pos[p]: the row of pair p; row_src[row]: the pair of a row (-1: padding);
// tile_expert[i]: the expert of tile i (-1: unused). Which of an expert's rows a pair gets depends on the order in which
// the threads arrive; a row's result does not depend on where it lies.
constexpr int PLAN_THREADS = 1024;
__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ ids, int P, int E, int tile, int max_tiles, int* __restrict__ pos, int* __restrict__ row_src,
                int* __restrict__ tile_expert) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ int sh[];                        // counts [E], first tile [E + 1]
    int* counts = sh;
    int* first = sh + E;
    for (int e = threadIdx.x; e < E; e += PLAN_THREADS) counts[e] = 0;
    for (int i = threadIdx.x; i < max_tiles; i += PLAN_THREADS) tile_expert[i] = -1;
    for (int i = threadIdx.x; i < max_tiles * tile; i += PLAN_THREADS) row_src[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += PLAN_THREADS)                                              // the pair's rank in its expert
        pos[p] = ids[p] < E ? atomicAdd(&counts[ids[p]], 1) : -1;                                    // (an identity expert: no row)
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < E; ++e) { first[e] = t; t += (counts[e] + tile - 1) / tile; }
        first[E] = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += PLAN_THREADS)
        for (int i = first[e]; i < first[e + 1]; ++i) tile_expert[i] = e;
    for (int p = threadIdx.x; p < P; p += PLAN_THREADS) {
        if (ids[p] >= E) continue;
        const int row = first[ids[p]] * tile + pos[p];
        pos[p] = row;
        row_src[row] = p;
    }
}

// dst[row, :] = x[row_src[row] / div, :] (zeros where row_src is negative): the rows of a grouped product, 16 bytes a thread.
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ row_src, int div, uint4* __restrict__ dst,
                                   int rows, int vecs) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)rows * vecs; i += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / vecs), v = (int)(i % vecs);
        const int src = row_src[row];
        dst[i] = src >= 0 ? x[(size_t)(src / div) * vecs + v] : make_uint4(0, 0, 0, 0);
    }
}

// out[t, :] = (add ? out[t, :] : 0) + sum_k wts[t, k] * y[pos[t * top + k], :], k ascending; a pair without a row (pos < 0:
// an identity expert) takes x[t, :].
template <typename TX>
__global__ void moe_combine_rows_kernel(const float* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ wts, float* out,
                                        int top, int d, size_t count, int add, const TX* __restrict__ x) {
    bl_pdl_trigger();
    bl_pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / d, c = e % d;
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = pos[t * top + k];
            acc = fmaf(wts[t * top + k], row < 0 ? (x ? bl_load(x + t * d + c) : 0.f) : y[(size_t)row * d + c], acc);
        }
        out[e] = add ? out[e] + acc : acc;
    }
}

template <typename TX, typename TW, typename TO>
int launch_expert(const void* x, int x_div, const void* w, size_t stride, const int* ids, void* out, int P, int N, int K, int epi,
                  const float* act, int n_real, cudaStream_t s) {
    const dim3 grid((N + WARPS - 1) / WARPS, P);
    if (epi == BL_EPI_NONE)
        BL_CUDA(bl_launch_dependent(expert_gemm_plain_kernel<TX, TW, TO, BL_EPI_NONE>, grid, dim3(WARPS * 32), 0, s, (const TX*)x, x_div,
                                    (const TW*)w, stride, ids, (TO*)out, P, N, K, act, n_real));
    else if (epi == BL_EPI_SWIGLU)
        BL_CUDA(bl_launch_dependent(expert_gemm_plain_kernel<TX, TW, TO, BL_EPI_SWIGLU>, grid, dim3(WARPS * 32), 0, s, (const TX*)x, x_div,
                                    (const TW*)w, stride, ids, (TO*)out, P, N, K, act, n_real));
    else
        BL_FAIL("bl_expert_gemm_plain: epilogue %d is not built", epi);
    BL_CHECK_LAUNCH("bl_expert_gemm_plain");
    return 0;
}

}  // namespace

extern "C" int bl_moe_route(const float* z, int ldz, const void* correction, int corr_dtype, int T, int E, int top, int n_groups,
                            int keep, int* ids, float* wts, void* stream) {
    return bl_moe_route_ext(z, ldz, correction, corr_dtype, T, E, top, n_groups, keep, ids, wts, BL_SCORE_SIGMOID, 2, stream);
}

extern "C" int bl_moe_route_ext(const float* z, int ldz, const void* correction, int corr_dtype, int T, int E, int top, int n_groups,
                                int keep, int* ids, float* wts, int score_kind, int group_top, void* stream) {
    if (T <= 0) return 0;
    if ((score_kind != BL_SCORE_SIGMOID && score_kind != BL_SCORE_SOFTMAX) || (group_top != 1 && group_top != 2))
        BL_FAIL("bl_moe_route: scores of kind %d, groups scored by their %d largest", score_kind, group_top);
    if (E <= 0 || top <= 0 || n_groups <= 0 || keep <= 0 || E % n_groups != 0 || keep > n_groups || top > keep * (E / n_groups) || ldz < E)
        BL_FAIL("bl_moe_route: %d experts in %d groups, %d groups kept, %d chosen", E, n_groups, keep, top);
    const size_t smem = (size_t)(2 * E + 2 * n_groups) * sizeof(float);
    if (smem > 48 * 1024) BL_FAIL("bl_moe_route: %d experts are too many for shared memory", E);
    BL_CUDA(bl_launch_dependent(moe_route_kernel, dim3(T), dim3(32), smem, (cudaStream_t)stream, z, ldz, correction, corr_dtype, E, top,
                                n_groups, keep, ids, wts, score_kind, group_top));
    BL_CHECK_LAUNCH("bl_moe_route");
    return 0;
}

extern "C" int bl_expert_gemm_plain(const void* x, int x_dtype, int x_div, const void* w, int w_dtype, long long expert_stride,
                                    const int* ids, void* out, int out_dtype, int P, int N, int K, int epilogue, const float* act,
                                    void* stream) {
    return bl_expert_gemm_plain_some(x, x_dtype, x_div, w, w_dtype, expert_stride, ids, out, out_dtype, P, N, K, epilogue, act,
                                     0x7fffffff, stream);
}

// The same with identity experts: pairs whose expert number is n_real or more are skipped (their rows of out stay as they are).
extern "C" int bl_expert_gemm_plain_some(const void* x, int x_dtype, int x_div, const void* w, int w_dtype, long long expert_stride,
                                         const int* ids, void* out, int out_dtype, int P, int N, int K, int epilogue, const float* act,
                                         int n_real, void* stream) {
    if (P <= 0) return 0;
    if (N <= 0 || K <= 0 || x_div <= 0 || P > 65535 * 32) BL_FAIL("bl_expert_gemm_plain: bad sizes P=%d N=%d K=%d", P, N, K);
    if (P > 65535) {                                          // the grid's y: in slices
        const size_t xe = x_dtype == BL_F32 ? 4 : 2, oe = out_dtype == BL_F32 ? 4 : 2;
        const int step = 65535 / x_div * x_div;
        for (int p0 = 0; p0 < P; p0 += step) {
            const int n = P - p0 < step ? P - p0 : step;
            if (bl_expert_gemm_plain_some((const char*)x + (size_t)(p0 / x_div) * K * xe, x_dtype, x_div, w, w_dtype, expert_stride, ids + p0,
                                          (char*)out + (size_t)p0 * N * oe, out_dtype, n, N, K, epilogue, act, n_real, stream)) return 1;
        }
        return 0;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const size_t st = (size_t)expert_stride;
    if (x_dtype == BL_F32 && w_dtype == BL_F32 && out_dtype == BL_F32)
        return launch_expert<float, float, float>(x, x_div, w, st, ids, out, P, N, K, epilogue, act, n_real, s);
    if (x_dtype == BL_BF16 && w_dtype == BL_BF16 && out_dtype == BL_F32)
        return launch_expert<__nv_bfloat16, __nv_bfloat16, float>(x, x_div, w, st, ids, out, P, N, K, epilogue, act, n_real, s);
    if (x_dtype == BL_BF16 && w_dtype == BL_BF16 && out_dtype == BL_BF16)
        return launch_expert<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(x, x_div, w, st, ids, out, P, N, K, epilogue, act, n_real, s);
    BL_FAIL("bl_expert_gemm_plain: unsupported dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
}

extern "C" int bl_moe_combine(const float* y, const float* wts, float* out, int T, int top, int d, int add, void* stream) {
    return bl_moe_combine_some(y, wts, out, T, top, d, add, nullptr, 0, nullptr, BL_F32, stream);
}

// ids (null: none) and n_real: pairs of identity experts take x[t, :] (x [T, d], 32-bit or bfloat16) in the place of their row.
extern "C" int bl_moe_combine_some(const float* y, const float* wts, float* out, int T, int top, int d, int add, const int* ids,
                                   int n_real, const void* x, int x_dtype, void* stream) {
    if (T <= 0) return 0;
    if (top <= 0 || d <= 0) BL_FAIL("bl_moe_combine: bad sizes top=%d d=%d", top, d);
    if (ids && !x) BL_FAIL("bl_moe_combine: identity experts need the tokens' input rows");
    const size_t count = (size_t)T * d;
    const int blocks = (int)((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
    if (x_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, y, wts, out, top, d,
                                    count, add, ids, n_real, (const __nv_bfloat16*)x));
    else
        BL_CUDA(bl_launch_dependent(moe_combine_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, y, wts, out, top, d, count,
                                    add, ids, n_real, (const float*)x));
    BL_CHECK_LAUNCH("bl_moe_combine");
    return 0;
}

// Lays the pairs (token, chosen expert) out for the grouped product (see moe_plan_kernel). max_tiles >= ceil(P / tile) + E.
extern "C" int bl_moe_plan(const int* ids, int P, int E, int tile, int max_tiles, int* pos, int* row_src, int* tile_expert, void* stream) {
    if (P <= 0) return 0;
    if (E <= 0 || tile <= 0 || max_tiles < (P + tile - 1) / tile + E) BL_FAIL("bl_moe_plan: %d pairs, %d experts, %d tiles of %d", P, E, max_tiles, tile);
    const size_t smem = (size_t)(2 * E + 1) * sizeof(int);
    if (smem > 48 * 1024) BL_FAIL("bl_moe_plan: %d experts are too many for shared memory", E);
    BL_CUDA(bl_launch_dependent(moe_plan_kernel, dim3(1), dim3(PLAN_THREADS), smem, (cudaStream_t)stream, ids, P, E, tile, max_tiles, pos,
                                row_src, tile_expert));
    BL_CHECK_LAUNCH("bl_moe_plan");
    return 0;
}

// dst[row, :] = x[row_src[row] / div, :], zeros where row_src[row] < 0; rows of `cols` bfloat16 values, cols a multiple of 8.
extern "C" int bl_gather_rows(const void* x, const int* row_src, int div, void* dst, int rows, int cols, void* stream) {
    if (rows <= 0) return 0;
    if (cols <= 0 || cols % 8 != 0 || div <= 0 || (((uintptr_t)x | (uintptr_t)dst) & 15)) BL_FAIL("bl_gather_rows: rows of %d values", cols);
    const int vecs = cols / 8;
    const size_t n = (size_t)rows * vecs;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    BL_CUDA(bl_launch_dependent(gather_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const uint4*)x, row_src, div,
                                (uint4*)dst, rows, vecs));
    BL_CHECK_LAUNCH("bl_gather_rows");
    return 0;
}

extern "C" int bl_moe_combine_rows(const float* y, const int* pos, const float* wts, float* out, int T, int top, int d, int add,
                                   void* stream) {
    return bl_moe_combine_rows_some(y, pos, wts, out, T, top, d, add, nullptr, BL_F32, stream);
}

// x (null: none) [T, d], 32-bit or bfloat16: what a pair without a row (an identity expert) contributes.
extern "C" int bl_moe_combine_rows_some(const float* y, const int* pos, const float* wts, float* out, int T, int top, int d, int add,
                                        const void* x, int x_dtype, void* stream) {
    if (T <= 0) return 0;
    if (top <= 0 || d <= 0) BL_FAIL("bl_moe_combine_rows: bad sizes top=%d d=%d", top, d);
    const size_t count = (size_t)T * d;
    const int blocks = (int)((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
    if (x_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(moe_combine_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, y, pos, wts, out,
                                    top, d, count, add, (const __nv_bfloat16*)x));
    else
        BL_CUDA(bl_launch_dependent(moe_combine_rows_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, y, pos, wts, out, top, d,
                                    count, add, (const float*)x));
    BL_CHECK_LAUNCH("bl_moe_combine_rows");
    return 0;
}

extern "C" int bl_table_route(const int* table, const int* tokens, int T, int top, int* ids, float* wts, void* stream) {
    if (T <= 0) return 0;
    if (top <= 0) BL_FAIL("bl_table_route: %d experts a token", top);
    BL_CUDA(bl_launch_dependent(table_route_kernel, dim3((T * top + 127) / 128), dim3(128), 0, (cudaStream_t)stream, table, tokens, T, top, ids, wts));
    BL_CHECK_LAUNCH("bl_table_route");
    return 0;
}
