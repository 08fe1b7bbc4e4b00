// Attention whose keys and values are made from ONE small vector per token (a latent of `rank` values) and one rotated
// key part of `rot` values that all heads share. The cache holds rows [latent | rotated part] and nothing per head.
// With k_h = Uk_h c and v_h = Uv_h c the products with Uk and Uv move to the query's side:
//     score(t, h, j) = (Uk_h^T q_h(t)) . c_j + q_rot_h(t) . r_j          out_h(t) = Uv_h (sum_j p_j c_j)
// so every head of every token reads the same cached rows: keys of rank + rot values whose first `rank` values are also
// the values. This file has the plain kernels of that path (the 32-bit path and the twins of the fast kernels):
//   bl_latent_prep          RMS norms of the query latent and of the key/value latent, rotation of the shared key part,
//                           the write of [latent | rotated part] into the token's page
//   bl_head_gemm_plain      a product per head, out[t, h, :] = x[t, h, :] . W_h (strides say how W_h lies), optionally
//                           times the sigmoid of a gate per output
//   bl_rope_heads           rotation of a slice of every head of a row (pairs (j, j + half)), cos and sin times a factor
//   bl_latent_attention_plain   one warp per (token, head) over the cached rows, a window, a sink per head
// Norm statistics, angles, scores, the softmax and all sums are 32-bit; angle = float(position) * inv_freq[j].
#include "common.cuh"
#include "api.h"

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = 4;
constexpr int MAX_RANK = 1024;            // values a lane keeps of the plain attention's output: MAX_RANK / 32

__device__ __forceinline__ float block_sum(float v, float* part) {
    v = bl_warp_sum(v);
    __syncthreads();                                   // part may still be read from the call before
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    return (part[0] + part[1]) + (part[2] + part[3]);
}

template <typename TT>
__global__ void __launch_bounds__(THREADS)
latent_prep_kernel(const float* proj, int ld, int off_q, int q_rank, int off_kv, int rank, int rot_dim, int rot_half,
                   const void* __restrict__ qw, int qw_dtype, const void* __restrict__ kw, int kw_dtype, float eps,
                   const int* __restrict__ positions, const int* __restrict__ tok_req, const int* __restrict__ block_table,
                   int max_pages, int page_size, const float* __restrict__ inv_freq, float mscale, TT* __restrict__ cq,
                   TT* __restrict__ cache) {
    bl_pdl_trigger();
    bl_pdl_wait();
    __shared__ float part[4];
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    if (cq) {
        const float* z = row + off_q;
        float s = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += THREADS) s += z[i] * z[i];
        const float inv = 1.0f / sqrtf(block_sum(s, part) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += THREADS)
            bl_store(cq + (size_t)t * q_rank + i, z[i] * inv * bl_load_any(qw, qw_dtype, i));
    }
    if (cache) {
        const float* z = row + off_kv;
        float s = 0.f;
        for (int i = threadIdx.x; i < rank; i += THREADS) s += z[i] * z[i];
        const float inv = 1.0f / sqrtf(block_sum(s, part) / (float)rank + eps);
        const int pos = positions[t];
        const int page = block_table[(size_t)tok_req[t] * max_pages + pos / page_size];
        TT* dst = cache + ((size_t)page * page_size + pos % page_size) * (rank + rot_dim);
        for (int i = threadIdx.x; i < rank; i += THREADS) bl_store(dst + i, z[i] * inv * bl_load_any(kw, kw_dtype, i));
        for (int j = threadIdx.x; j < rot_half; j += THREADS) {
            const float a = (float)pos * inv_freq[j];
            const float c = cosf(a) * mscale, sn = sinf(a) * mscale;
            const float u = z[rank + j], v = z[rank + rot_half + j];
            bl_store(dst + rank + j, u * c - v * sn);
            bl_store(dst + rank + rot_half + j, v * c + u * sn);
        }
        for (int d = 2 * rot_half + threadIdx.x; d < rot_dim; d += THREADS) bl_store(dst + rank + d, z[rank + d]);   // not rotated
    }
}

// out[t, h, n] = sum_k x[t, h, k] * W[h][n, k], W[h][n, k] at w + h * w_head + n * w_n + k * w_k; one FMA chain per
// output in ascending k. x and out are 32-bit or bfloat16 by a run-time code, W by the template.
template <typename TW>
__global__ void __launch_bounds__(THREADS)
head_gemm_plain_kernel(const void* x, int x_dtype, size_t ldx, size_t x_head, const TW* __restrict__ w, size_t w_head, size_t w_n,
                       size_t w_k, void* out, int out_dtype, size_t ld_out, size_t out_head, int N, int K, const float* gate,
                       size_t ld_gate) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ float xs[];
    const int h = blockIdx.y, t = blockIdx.z;
    for (int k = threadIdx.x; k < K; k += THREADS) xs[k] = bl_load_any(x, x_dtype, (size_t)t * ldx + (size_t)h * x_head + k);
    __syncthreads();
    const int n = blockIdx.x * THREADS + threadIdx.x;
    if (n >= N) return;
    const TW* wr = w + (size_t)h * w_head + (size_t)n * w_n;
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc = fmaf(xs[k], bl_load(wr + (size_t)k * w_k), acc);
    if (gate) acc *= 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate + (size_t)h * N + n]));
    const size_t o = (size_t)t * ld_out + (size_t)h * out_head + n;
    if (out_dtype == BL_F32) ((float*)out)[o] = acc;
    else ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(acc);
}

template <typename TO>
__global__ void __launch_bounds__(THREADS)
rope_heads_kernel(const float* q, size_t ld, size_t head_stride, int off, const int* __restrict__ positions,
                  const float* __restrict__ inv_freq, int n, int rot_half, float mscale, TO* __restrict__ out, size_t ld_out,
                  size_t out_head, int out_off, int H, const float* lead, int n_lead, TO* __restrict__ lead_out, size_t ld_lead,
                  size_t lead_head) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ float cs[];                      // cos [rot_half], sin [rot_half]
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int j = threadIdx.x; j < rot_half; j += THREADS) {
        const float a = (float)pos * inv_freq[j];
        cs[j] = cosf(a) * mscale;
        cs[rot_half + j] = sinf(a) * mscale;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < H * rot_half; e += THREADS) {
        const int h = e / rot_half, j = e % rot_half;
        const float* src = q + (size_t)t * ld + (size_t)h * head_stride + off;
        TO* dst = out + (size_t)t * ld_out + (size_t)h * out_head + out_off;
        const float u = src[j], v = src[rot_half + j];
        bl_store(dst + j, u * cs[j] - v * cs[rot_half + j]);
        bl_store(dst + rot_half + j, v * cs[j] + u * cs[rot_half + j]);
    }
    const int rest = n - 2 * rot_half;                 // values of a head's slice that are not rotated
    for (int e = threadIdx.x; e < H * rest; e += THREADS) {
        const int h = e / rest, d = 2 * rot_half + e % rest;
        bl_store(out + (size_t)t * ld_out + (size_t)h * out_head + out_off + d, q[(size_t)t * ld + (size_t)h * head_stride + off + d]);
    }
    // another slice of every head (the part of q that is not rotated), strided as q, cast into a tensor of its own
    for (int e = threadIdx.x; e < H * n_lead; e += THREADS) {
        const int h = e / n_lead, d = e % n_lead;
        bl_store(lead_out + (size_t)t * ld_lead + (size_t)h * lead_head + d, lead[(size_t)t * ld + (size_t)h * head_stride + d]);
    }
}

template <typename TT>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_plain_kernel(const TT* __restrict__ q, const TT* __restrict__ cache, const int* __restrict__ tok_req,
                              const int* __restrict__ cu_q, const int* __restrict__ ctx_len, const int* __restrict__ block_table,
                              int max_pages, TT* __restrict__ out, int T, int H, int dk, int dv, int page_size, int window,
                              float scale, const void* __restrict__ sinks, int sink_dtype) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ float qs_all[];                  // [WARPS][dk]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + warp;
    if (item >= T * H) return;                         // whole warps leave together; no block-wide barrier below
    float* qs = qs_all + (size_t)warp * dk;
    const int t = item / H, h = item % H;
    const int r = tok_req[t];
    const int q_len = cu_q[r + 1] - cu_q[r];
    const int pos = ctx_len[r] - q_len + (t - cu_q[r]);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const TT* qrow = q + ((size_t)t * H + h) * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = bl_load(qrow + d);
    __syncwarp();
    const int* bt = block_table + (size_t)r * max_pages;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_RANK / 32];
#pragma unroll
    for (int i = 0; i < MAX_RANK / 32; ++i) acc[i] = 0.f;
    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        const bool valid = j <= pos;
        float s = -INFINITY;
        if (valid) {
            const TT* krow = cache + ((size_t)bt[j / page_size] * page_size + j % page_size) * dk;
            float dot = 0.f;
            for (int d = 0; d < dk; ++d) dot = fmaf(qs[d], bl_load(krow + d), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, bl_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);           // first chunk: exp(-inf) = 0
        l = l * alpha + bl_warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_RANK / 32; ++i) acc[i] *= alpha;
        const int n = min(32, pos - base + 1);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int key = base + jj;
            const TT* vrow = cache + ((size_t)bt[key / page_size] * page_size + key % page_size) * dk;
#pragma unroll
            for (int i = 0; i < MAX_RANK / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, bl_load(vrow + d), acc[i]);
            }
        }
        m = m_new;
    }
    if (sinks) {                                       // one more term of the denominator, after the last key
        const float sk = bl_load_any(sinks, sink_dtype, h);
        const float m_new = fmaxf(m, sk);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < MAX_RANK / 32; ++i) acc[i] *= alpha;
    }
    TT* orow = out + ((size_t)t * H + h) * dv;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_RANK / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) bl_store(orow + d, acc[i] * inv);
    }
}

// tile[i] = i / per: the matrix (head) of each tile of 128 rows when every head has `per` tiles.
__global__ void head_tiles_kernel(int* __restrict__ tile, int n, int per) {
    bl_pdl_trigger();
    bl_pdl_wait();                    // every kernel of a step waits, or its successor could overtake the kernel before it
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) tile[i] = i / per;
}

// out[t, h * N + n] = hv[h, t, n] * sigmoid(gate[t, h * N + n]): head-major 32-bit sums back to token rows, gated.
template <typename TO>
__global__ void heads_gate_rows_kernel(const float* __restrict__ hv, const float* gate, size_t ld_gate, TO* __restrict__ out, int T, int H,
                                       int N, size_t Tp) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const size_t total = (size_t)T * H * N;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / ((size_t)H * N), c = e % ((size_t)H * N);
        const size_t h = c / N, n = c % N;
        float v = hv[(h * Tp + t) * N + n];
        if (gate) v *= 1.0f / (1.0f + expf(-gate[t * ld_gate + c]));
        bl_store(out + e, v);
    }
}

}  // namespace

extern "C" int bl_head_tiles(int* tile, int n_heads, int per, void* stream) {
    if (n_heads <= 0 || per <= 0) BL_FAIL("bl_head_tiles: %d heads with %d tiles each", n_heads, per);
    const int n = n_heads * per;
    BL_CUDA(bl_launch_dependent(head_tiles_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, tile, n, per));
    BL_CHECK_LAUNCH("bl_head_tiles");
    return 0;
}

extern "C" int bl_heads_gate_rows(const float* hv, const float* gate, long long ld_gate, void* out, int out_dtype, int T, int H, int N,
                                  int Tp, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || N <= 0 || Tp < T) BL_FAIL("bl_heads_gate_rows: bad sizes T=%d H=%d N=%d Tp=%d", T, H, N, Tp);
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)T * H * N;
    const int g = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (out_dtype == BL_F32) BL_CUDA(bl_launch_dependent(heads_gate_rows_kernel<float>, dim3(g), dim3(256), 0, s, hv, gate, (size_t)ld_gate, (float*)out, T, H, N, (size_t)Tp));
    else if (out_dtype == BL_BF16) BL_CUDA(bl_launch_dependent(heads_gate_rows_kernel<__nv_bfloat16>, dim3(g), dim3(256), 0, s, hv, gate, (size_t)ld_gate, (__nv_bfloat16*)out, T, H, N, (size_t)Tp));
    else BL_FAIL("bl_heads_gate_rows: unknown dtype %d", out_dtype);
    BL_CHECK_LAUNCH("bl_heads_gate_rows");
    return 0;
}

extern "C" int bl_latent_prep(const float* proj, int ld, int off_q, int q_rank, int off_kv, int rank, int rot_dim, int rot_half,
                              const void* q_norm_w, int qw_dtype, const void* kv_norm_w, int kw_dtype, float eps,
                              const int* positions, const int* tok_req, const int* block_table, int max_pages, int page_size,
                              const float* inv_freq, float mscale, void* cq, void* cache, int dtype, int T, void* stream) {
    if (T <= 0) return 0;
    if (cq && (q_rank <= 0 || off_q < 0 || off_q + q_rank > ld || !q_norm_w))
        BL_FAIL("bl_latent_prep: the query latent (%d values from column %d) does not fit rows of %d", q_rank, off_q, ld);
    if (cache && (rank <= 0 || rot_half < 0 || 2 * rot_half > rot_dim || off_kv < 0 || off_kv + rank + rot_dim > ld || !kv_norm_w || page_size <= 0 || max_pages <= 0))
        BL_FAIL("bl_latent_prep: the key/value latent (%d + %d values from column %d, %d pairs rotated) does not fit rows of %d", rank, rot_dim, off_kv, rot_half, ld);
    cudaStream_t s = (cudaStream_t)stream;
#define BL_GO(TT) BL_CUDA(bl_launch_dependent(latent_prep_kernel<TT>, dim3(T), dim3(THREADS), 0, s, proj, ld, off_q, q_rank, off_kv, rank, \
        rot_dim, rot_half, q_norm_w, qw_dtype, kv_norm_w, kw_dtype, eps, positions, tok_req, block_table, max_pages, page_size, inv_freq, mscale, \
        (TT*)cq, (TT*)cache))
    if (dtype == BL_F32) BL_GO(float);
    else if (dtype == BL_BF16) BL_GO(__nv_bfloat16);
    else BL_FAIL("bl_latent_prep: unknown dtype %d", dtype);
#undef BL_GO
    BL_CHECK_LAUNCH("bl_latent_prep");
    return 0;
}

extern "C" int bl_head_gemm_plain(const void* x, int x_dtype, long long ldx, long long x_head, const void* w, int w_dtype,
                                  long long w_head, long long w_n, long long w_k, void* out, int out_dtype, long long ld_out,
                                  long long out_head, int T, int H, int N, int K, const float* gate, long long ld_gate, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || N <= 0 || K <= 0 || K > 12000) BL_FAIL("bl_head_gemm_plain: bad sizes H=%d N=%d K=%d", H, N, K);
    if (H > 65535 || T > 65535) BL_FAIL("bl_head_gemm_plain: %d heads and %d rows exceed the grid", H, T);
    if ((x_dtype != BL_F32 && x_dtype != BL_BF16) || (out_dtype != BL_F32 && out_dtype != BL_BF16))
        BL_FAIL("bl_head_gemm_plain: unknown dtype %d / %d", x_dtype, out_dtype);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((N + THREADS - 1) / THREADS, H, T);
    const size_t smem = (size_t)K * sizeof(float);
#define BL_GO(TW) BL_CUDA(bl_launch_dependent(head_gemm_plain_kernel<TW>, grid, dim3(THREADS), smem, s, x, x_dtype, (size_t)ldx, (size_t)x_head, \
        (const TW*)w, (size_t)w_head, (size_t)w_n, (size_t)w_k, out, out_dtype, (size_t)ld_out, (size_t)out_head, N, K, gate, (size_t)ld_gate))
    if (w_dtype == BL_F32) BL_GO(float);
    else if (w_dtype == BL_BF16) BL_GO(__nv_bfloat16);
    else BL_FAIL("bl_head_gemm_plain: unknown weight dtype %d", w_dtype);
#undef BL_GO
    BL_CHECK_LAUNCH("bl_head_gemm_plain");
    return 0;
}

extern "C" int bl_rope_heads(const float* q, long long ld, long long head_stride, int off, const int* positions,
                             const float* inv_freq, int n, int rot_half, float mscale, void* out, int out_dtype, long long ld_out,
                             long long out_head, int out_off, int T, int H, const float* lead, int n_lead, void* lead_out,
                             long long ld_lead, long long lead_head, void* stream) {
    if (T <= 0 || n <= 0) return 0;
    if (n_lead < 0 || (n_lead > 0 && (lead == nullptr || lead_out == nullptr))) BL_FAIL("bl_rope_heads: a second slice of %d values without its tensors", n_lead);
    if (H <= 0 || off < 0 || out_off < 0 || rot_half < 0 || 2 * rot_half > n) BL_FAIL("bl_rope_heads: bad sizes H=%d n=%d pairs=%d offsets %d, %d", H, n, rot_half, off, out_off);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(2 * rot_half + 1) * sizeof(float);
#define BL_GO(TO) BL_CUDA(bl_launch_dependent(rope_heads_kernel<TO>, dim3(T), dim3(THREADS), smem, s, q, (size_t)ld, (size_t)head_stride, off, \
        positions, inv_freq, n, rot_half, mscale, (TO*)out, (size_t)ld_out, (size_t)out_head, out_off, H, lead, n_lead, (TO*)lead_out, \
        (size_t)ld_lead, (size_t)lead_head))
    if (out_dtype == BL_F32) BL_GO(float);
    else if (out_dtype == BL_BF16) BL_GO(__nv_bfloat16);
    else BL_FAIL("bl_rope_heads: unknown dtype %d", out_dtype);
#undef BL_GO
    BL_CHECK_LAUNCH("bl_rope_heads");
    return 0;
}

extern "C" int bl_latent_attention_plain(const void* q, const void* cache, int dtype, const int* tok_req, const int* cu_q,
                                         const int* ctx_len, const int* block_table, int max_pages, void* out, int T, int H,
                                         int dk, int dv, int page_size, int window, float scale, const void* sinks,
                                         int sink_dtype, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || dv > dk || dv > MAX_RANK || dk > 2 * MAX_RANK)
        BL_FAIL("bl_latent_attention_plain: keys of %d and values of %d (the keys' first) are outside what this kernel holds (%d)", dk, dv, MAX_RANK);
    if (page_size <= 0 || max_pages <= 0 || window < 0) BL_FAIL("bl_latent_attention_plain: bad page size, table width or window");
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (T * H + WARPS - 1) / WARPS;
    const size_t smem = (size_t)WARPS * dk * sizeof(float);
#define BL_GO(TT) BL_CUDA(bl_launch_dependent(latent_attention_plain_kernel<TT>, dim3(blocks), dim3(WARPS * 32), smem, s, (const TT*)q, \
        (const TT*)cache, tok_req, cu_q, ctx_len, block_table, max_pages, (TT*)out, T, H, dk, dv, page_size, window, scale, sinks, sink_dtype))
    if (dtype == BL_F32) BL_GO(float);
    else if (dtype == BL_BF16) BL_GO(__nv_bfloat16);
    else BL_FAIL("bl_latent_attention_plain: unknown dtype %d", dtype);
#undef BL_GO
    BL_CHECK_LAUNCH("bl_latent_attention_plain");
    return 0;
}
