// Attention over one cached latent per token on tensor cores (bfloat16 operands, 32-bit scores, softmax and sums).
// The cache holds rows [latent (rank) | rotated key part (rot)]; the queries have been moved into the latent's space, so
// every head of every token reads the same rows: keys of dk = rank + rot values whose first `rank` values are the values.
// Queries and results lie HEAD-MAJOR, [H, Tp, .] with Tp the step's tokens rounded up to the grouped product's tile, so
// that the products with the heads' own matrices before and after run as one grouped product each.
//
// A block is 32 rows and 8 warps. With several new tokens in a request the rows are 32 consecutive tokens of one head;
// for a request with a single token they are up to 32 of its heads. The block walks the visible keys in blocks of 64,
// double-buffered through cp.async. Per key block:
//   scores: warp (row group rg, quarter qt) multiplies its 16 rows by the 16 keys of its quarter over all of dk and
//           leaves the raw 32-bit scores in shared memory;
//   softmax: warp w owns rows 4w .. 4w + 3 (eight lanes a row): mask, running maximum and sum, and the weights, which
//           it writes as bfloat16 into the place of the row's scores beside the factor for the row's sums so far (no
//           exponential is computed twice);
//   values: warp (rg, qt) scales its sums by the factors of its 16 rows, fetches the weights as the left operand and
//           multiplies them by its own quarter of the value columns, up to NTW tiles of 8 columns.
// Each phase has the tensor-core work split four ways without any product computed twice; the output of 16 rows x 512
// value columns, which no warp could hold, is 64 registers a thread. A sink per head joins the denominator at the end.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int PAGE = 16;
constexpr int KB = 64;            // keys per block
constexpr int ROWS = 32;          // rows per thread block
constexpr int THREADS = 256;
constexpr int PAD = 8;            // bfloat16 elements of padding per shared-memory row (keeps ldmatrix conflict-free)
constexpr int SROW = KB + 4;      // floats per row of the score buffer

struct LatentParams {
    const __nv_bfloat16* q_lat; const __nv_bfloat16* q_rot; const __nv_bfloat16* cache; __nv_bfloat16* out;
    const int* cu_q; const int* ctx_len; const int* block_table; int max_pages;
    const int* work;              // several tokens: [n][2] (request, first token of a 64-token tile); single: [n] requests
    int H, Tp, rank, rot, window;
    float scale_log2;
    const void* sinks; int sink_dtype;
    // single tokens with a long context: the key blocks are cut into n_splits slices, one block each, which leave their
    // unnormalised result, maximum and sum here ([requests * H][n_splits][rank] and [..][2]) for the merge kernel
    float* part_o; float* part_ml; int n_splits;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(addr), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Keys [key0, key0 + 64) into a stage of rows `row` elements apart. The 16 rows of a page lie together, dk values each.
// Pages outside [lo, hi] or no longer in the table, and keys past hi, become zeros: they are masked anyway, and zeros keep
// the value product finite whatever an earlier request left in a page that is used again.
__device__ __forceinline__ void load_keys(__nv_bfloat16* stage, int row, const LatentParams& p, const int* table, int dk,
                                          int key0, int lo, int hi) {
    const int ch = dk / 8;                                        // 16-byte chunks per row
    const int c0 = threadIdx.x & 7;                               // eight threads a row, 32 rows a pass: no division by ch
#pragma unroll
    for (int r = threadIdx.x >> 3; r < KB; r += THREADS / 8) {
        const int key = key0 + r;
        const int first = key - key % PAGE;
        const int page = (first + PAGE - 1 >= lo && key <= hi) ? table[key / PAGE] : -1;
        __nv_bfloat16* dst = stage + r * row;
        if (page >= 0) {
            const __nv_bfloat16* src = p.cache + ((size_t)page * PAGE + key % PAGE) * dk;
            for (int c = c0; c < ch; c += 8) cp_async16(dst + c * 8, src + c * 8);
        } else {
            for (int c = c0; c < ch; c += 8) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}

template <int NTW, bool SINGLE>
__global__ void __launch_bounds__(THREADS, NTW <= 8 ? 2 : 1)
latent_attention_mma_kernel(const LatentParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk = p.rank + p.rot;
    const int dkp = (dk + 15) & ~15;
    const int row = dkp + PAD;
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [ROWS][row]
    __nv_bfloat16* ks = qs + ROWS * row;                                      // [2][KB][row]
    float* ss = reinterpret_cast<float*>(ks + 2 * KB * row);                  // [ROWS][SROW]: scores, then the weights in their place
    float* fac = ss + ROWS * SROW;                                            // [2][ROWS]: a row's factor for its sums so far; its last factor
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int rg = warp >> 2, qt = warp & 3;
    const int mi = lane >> 3, ri = lane & 7;                      // ldmatrix: which 8x8 matrix, which row of it
    bl_pdl_trigger();
    int r, tok0, head0, item = 0, split = 0;
    if (SINGLE) {
        const int per = (p.H + ROWS - 1) / ROWS;
        const int unit = blockIdx.x / p.n_splits;
        split = blockIdx.x % p.n_splits;
        item = unit / per;
        r = p.work[item];
        tok0 = 0;
        head0 = (unit % per) * ROWS;
    } else {
        // all heads of the last tile first: late tiles of a request see the most keys
        const int unit = gridDim.x / p.H - 1 - blockIdx.x / p.H;
        r = p.work[2 * (unit >> 1)];
        tok0 = p.work[2 * (unit >> 1) + 1] + (unit & 1) * ROWS;
        head0 = blockIdx.x % p.H;
    }
    const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin, ctx = p.ctx_len[r];
    const int* table = p.block_table + (size_t)r * p.max_pages;
    const int n_rows = SINGLE ? (q_len > 0 ? min(ROWS, p.H - head0) : 0) : max(0, min(ROWS, q_len - tok0));
    if (n_rows <= 0) {                                            // the whole block leaves together
        bl_pdl_wait();                                            // (a launch whose blocks all left without waiting would let its successor overtake)
        return;
    }
    // the padding columns of the operands are zero once and for all (the copies never touch them)
    for (int i = threadIdx.x; i < (ROWS + 2 * KB) * (row - dk); i += THREADS) {
        const int rr = i / (row - dk), c = dk + i % (row - dk);
        qs[rr * row + c] = __float2bfloat16_rn(0.f);
    }
    const int p_first = ctx - q_len + tok0;
    const int p_last = SINGLE ? p_first : p_first + n_rows - 1;
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    const int hi = p_last;
    int b_begin = lo / KB, b_end = hi / KB + 1;
    if (SINGLE && p.n_splits > 1) {
        const int each = (b_end - b_begin + p.n_splits - 1) / p.n_splits;
        b_begin = min(b_begin + split * each, b_end);
        b_end = min(b_begin + each, b_end);
    }
    bl_pdl_wait();                                                // queries and the newest rows of the cache come from kernels before
    {
        const int chl = p.rank / 8, ch = dk / 8;
        for (int i = threadIdx.x; i < ROWS * ch; i += THREADS) {
            const int rr = i / ch, c = i % ch;
            __nv_bfloat16* dst = qs + rr * row + c * 8;
            if (rr < n_rows) {
                const size_t at = (size_t)(SINGLE ? head0 + rr : head0) * p.Tp + (size_t)(q_begin + (SINGLE ? tok0 : tok0 + rr));
                const __nv_bfloat16* src = c < chl ? p.q_lat + at * p.rank + c * 8 : p.q_rot + at * p.rot + (c - chl) * 8;
                cp_async16(dst, src);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
    if (b_begin < b_end) load_keys(ks, row, p, table, dk, b_begin * KB, lo, hi);
    cp_async_commit();
    // The softmax of a row belongs to ONE warp: warp w owns rows 4w .. 4w + 3, eight lanes a row, eight keys a lane. It keeps
    // the row's maximum and sum, and leaves the weights (bfloat16, in the place of the row's scores) and the factor for the
    // sums so far in shared memory, where the warps of the row's group fetch them as the left operand of the value product.
    const int own = warp * 4 + (lane >> 3), sub = lane & 7;
    const int pos = own < n_rows ? (SINGLE ? p_first : p_first + own) : -1;   // a row that is no query sees nothing
    const int lo_row = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    float o[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m = -INFINITY, l = 0.f;
    const int v_cols = (p.rank + 15) & ~15;                       // value columns in pairs of tiles
    for (int b = b_begin; b < b_end; ++b) {
        __nv_bfloat16* stage = ks + ((b - b_begin) & 1) * KB * row;
        cp_async_wait_all();
        __syncthreads();                                          // block b has landed; everybody is through with block b - 1
        if (b + 1 < b_end) {
            load_keys(ks + ((b + 1 - b_begin) & 1) * KB * row, row, p, table, dk, (b + 1) * KB, lo, hi);
            cp_async_commit();
        }
        {   // scores of 16 rows x the 16 keys of this warp's quarter
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 2
            for (int kk = 0; kk < dkp / 16; ++kk) {
                unsigned a[4], bf[4];
                ldmatrix_x4(a, qs + (rg * 16 + (mi & 1) * 8 + ri) * row + kk * 16 + (mi >> 1) * 8);
                ldmatrix_x4(bf, stage + (qt * 16 + (mi >> 1) * 8 + ri) * row + kk * 16 + (mi & 1) * 8);
                mma_bf16(s[0], a, bf[0], bf[1]);
                mma_bf16(s[1], a, bf[2], bf[3]);
            }
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                float* d0 = ss + (rg * 16 + g) * SROW + qt * 16 + n * 8 + 2 * t;
                *reinterpret_cast<float2*>(d0) = make_float2(s[n][0], s[n][1]);
                *reinterpret_cast<float2*>(d0 + 8 * SROW) = make_float2(s[n][2], s[n][3]);
            }
        }
        __syncthreads();
        {   // the owner's pass over its row: mask, maximum, weights, sum
            float* srow = ss + own * SROW + sub * 8;
            const float4 u = *reinterpret_cast<const float4*>(srow), v = *reinterpret_cast<const float4*>(srow + 4);
            float e[8] = {u.x, u.y, u.z, u.w, v.x, v.y, v.z, v.w};
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int j = b * KB + sub * 8 + c;
                e[c] = (j <= pos && j >= lo_row) ? e[c] : -INFINITY;
                mx = fmaxf(mx, e[c]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_new = fmaxf(m, mx * p.scale_log2);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;             // a row that has seen no key yet
            const float alpha = ex2(m - m_use);                               // 2^-inf = 0 on the first block
            m = m_new;
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                e[c] = ex2(fmaf(e[c], p.scale_log2, -m_use));                 // a masked score is -inf: 2^-inf = 0
                part += e[c];
            }
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            part += __shfl_xor_sync(0xffffffffu, part, 4);
            l = l * alpha + part;
            __syncwarp();                                                     // the row's scores have been read: its weights take their place
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(ss + own * SROW) + sub * 8) =
                make_uint4(pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]), pack_bf16(e[4], e[5]), pack_bf16(e[6], e[7]));
            if (sub == 0) fac[own] = alpha;
        }
        __syncthreads();
        {
            const float a0 = fac[rg * 16 + g], a1 = fac[rg * 16 + g + 8];
            if (a0 != 1.f || a1 != 1.f) {
#pragma unroll
                for (int n = 0; n < NTW; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
            }
        }
        // out += P . V over this warp's value columns, P rounded to bfloat16 as the tensor cores' left operand
        const __nv_bfloat16* ps = reinterpret_cast<const __nv_bfloat16*>(ss);
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
            unsigned a[4];
            ldmatrix_x4(a, ps + (rg * 16 + (mi & 1) * 8 + ri) * (2 * SROW) + kk * 16 + (mi >> 1) * 8);
#pragma unroll
            for (int np = 0; np < NTW / 2; ++np) {
                const int col = (qt * NTW + 2 * np) * 8;
                if (col < v_cols) {
                    unsigned bf[4];
                    ldmatrix_x4_trans(bf, stage + (kk * 16 + (mi & 1) * 8 + ri) * row + col + (mi >> 1) * 8);
                    mma_bf16(o[2 * np], a, bf[0], bf[1]);
                    mma_bf16(o[2 * np + 1], a, bf[2], bf[3]);
                }
            }
        }
    }
    cp_async_wait_all();                                          // (a slice without key blocks has only asked for its queries)
    if (SINGLE && p.n_splits > 1) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int rr = rg * 16 + g + 8 * h;
            if (rr >= n_rows) continue;
            const size_t prow = ((size_t)item * p.H + head0 + rr) * p.n_splits + split;
            float* po = p.part_o + prow * p.rank;
#pragma unroll
            for (int n = 0; n < NTW; ++n) {
                const int col = (qt * NTW + n) * 8 + 2 * t;
                if (col < p.rank) *reinterpret_cast<float2*>(po + col) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
            }
        }
        if (sub == 0 && own < n_rows) {
            const size_t prow = ((size_t)item * p.H + head0 + own) * p.n_splits + split;
            p.part_ml[2 * prow] = m;
            p.part_ml[2 * prow + 1] = l;
        }
        return;
    }
    if (sub == 0 && own < n_rows) {
        float f = 1.f, den = l;
        if (p.sinks) {                                            // one more term of the denominator: unscaled, no value
            const float sk = bl_load_any(p.sinks, p.sink_dtype, SINGLE ? head0 + own : head0) * 1.4426950408889634f;
            const float mm = fmaxf(m, sk);
            f = exp2f(m - mm);
            den = den * f + exp2f(sk - mm);
        }
        fac[ROWS + own] = den > 0.f ? f / den : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int rr = rg * 16 + g + 8 * h;
        if (rr >= n_rows) continue;
        const int head = SINGLE ? head0 + rr : head0;
        const float inv = fac[ROWS + rr];
        const size_t at = (size_t)head * p.Tp + (size_t)(q_begin + (SINGLE ? tok0 : tok0 + rr));
        __nv_bfloat16* dst = p.out + at * p.rank;
#pragma unroll
        for (int n = 0; n < NTW; ++n) {
            const int col = (qt * NTW + n) * 8 + 2 * t;
            if (col < p.rank) *reinterpret_cast<unsigned*>(dst + col) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
        }
    }
}

// The slices of one (request, head): out = sum_s o_s 2^(m_s - M) / (sum_s l_s 2^(m_s - M) + 2^(sink - M)), in slice order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const LatentParams p) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int item = blockIdx.x / p.H, head = blockIdx.x % p.H;
    const int r = p.work[item];
    const int q_begin = p.cu_q[r];
    if (p.cu_q[r + 1] - q_begin <= 0) return;
    const size_t prow = ((size_t)item * p.H + head) * p.n_splits;
    float mm = -INFINITY;
    for (int s = 0; s < p.n_splits; ++s) mm = fmaxf(mm, p.part_ml[2 * (prow + s)]);
    float sk = -INFINITY;
    if (p.sinks) { sk = bl_load_any(p.sinks, p.sink_dtype, head) * 1.4426950408889634f; mm = fmaxf(mm, sk); }
    float den = p.sinks ? exp2f(sk - mm) : 0.f;
    for (int s = 0; s < p.n_splits; ++s) {
        const float ms = p.part_ml[2 * (prow + s)];
        if (ms != -INFINITY) den += p.part_ml[2 * (prow + s) + 1] * exp2f(ms - mm);
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    __nv_bfloat16* dst = p.out + ((size_t)head * p.Tp + q_begin) * p.rank;
    for (int c = threadIdx.x; c < p.rank; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float ms = p.part_ml[2 * (prow + s)];
            if (ms != -INFINITY) acc += p.part_o[(prow + s) * p.rank + c] * exp2f(ms - mm);
        }
        dst[c] = __float2bfloat16_rn(acc * inv);
    }
}

size_t smem_bytes(int dk) {
    const int row = ((dk + 15) & ~15) + PAD;
    return (size_t)(ROWS + 2 * KB) * row * sizeof(__nv_bfloat16) + (size_t)ROWS * (SROW + 2) * sizeof(float);
}

template <int NTW, bool SINGLE>
int launch(const LatentParams& p, int blocks, cudaStream_t s) {
    const size_t bytes = smem_bytes(p.rank + p.rot);
    static thread_local size_t allowed = 0;
    if (bytes > allowed) {
        BL_CUDA(cudaFuncSetAttribute(latent_attention_mma_kernel<NTW, SINGLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        allowed = bytes;
    }
    BL_CUDA(bl_launch_dependent(latent_attention_mma_kernel<NTW, SINGLE>, dim3(blocks), dim3(THREADS), bytes, s, p));
    BL_CHECK_LAUNCH("bl_latent_attention_mma");
    return 0;
}

}  // namespace

extern "C" int bl_latent_attention_mma_supported(int rank, int rot, int page_size) {
    return page_size == PAGE && rank > 0 && rot >= 0 && rank % 8 == 0 && rot % 8 == 0 && rank <= 512 && smem_bytes(rank + rot) <= 227 * 1024;
}

extern "C" int bl_latent_attention_mma(const void* q_lat, const void* q_rot, const void* cache, const int* cu_q, const int* ctx_len,
                                       const int* block_table, int max_pages, const int* work, int n_work, int single, void* out,
                                       int H, int Tp, int rank, int rot, int page_size, int window, float scale, const void* sinks,
                                       int sink_dtype, int n_splits, float* part_o, float* part_ml, void* stream) {
    if (n_work <= 0) return 0;
    if (!bl_latent_attention_mma_supported(rank, rot, page_size))
        BL_FAIL("bl_latent_attention_mma: rows of %d + %d values in pages of %d are not what this kernel is built for", rank, rot, page_size);
    if (H <= 0 || Tp <= 0 || max_pages <= 0 || window < 0) BL_FAIL("bl_latent_attention_mma: bad sizes H=%d Tp=%d", H, Tp);
    if ((((uintptr_t)q_lat | (uintptr_t)q_rot | (uintptr_t)cache | (uintptr_t)out) & 15) != 0)
        BL_FAIL("bl_latent_attention_mma: queries, cache and output must be 16-byte aligned");
    LatentParams p;
    p.q_lat = (const __nv_bfloat16*)q_lat; p.q_rot = (const __nv_bfloat16*)q_rot; p.cache = (const __nv_bfloat16*)cache;
    p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_pages = max_pages;
    p.work = work; p.H = H; p.Tp = Tp; p.rank = rank; p.rot = rot; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.sinks = sinks; p.sink_dtype = sink_dtype;
    if (!single || n_splits < 1) n_splits = 1;
    if (n_splits > 1 && (!part_o || !part_ml)) BL_FAIL("bl_latent_attention_mma: %d slices need scratch memory", n_splits);
    p.n_splits = n_splits; p.part_o = part_o; p.part_ml = part_ml;
    cudaStream_t s = (cudaStream_t)stream;
    const long long blocks = single ? (long long)n_work * ((H + ROWS - 1) / ROWS) * n_splits : (long long)n_work * 2 * H;
    if (blocks > 0x7fffffffLL) BL_FAIL("bl_latent_attention_mma: too many blocks");
    const int tiles = (rank + 7) / 8;                             // value tiles of 8 columns, dealt to four warps in even numbers
    int rc;
    if (tiles <= 16) rc = single ? launch<4, true>(p, (int)blocks, s) : launch<4, false>(p, (int)blocks, s);
    else if (tiles <= 32) rc = single ? launch<8, true>(p, (int)blocks, s) : launch<8, false>(p, (int)blocks, s);
    else rc = single ? launch<16, true>(p, (int)blocks, s) : launch<16, false>(p, (int)blocks, s);
    if (rc || n_splits == 1) return rc;
    BL_CUDA(bl_launch_dependent(latent_merge_kernel, dim3(n_work * H), dim3(128), 0, s, p));
    BL_CHECK_LAUNCH("bl_latent_attention_mma (merge)");
    return 0;
}
