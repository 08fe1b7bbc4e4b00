// Linear recurrences with a matrix state per head, S [key channels, value channels], carried per request in a state
// slot, for prompts' portions and single decoded tokens alike (a request's tokens are cu_q[r] .. cu_q[r + 1] - 1 of
// the batch; a request without tokens is left alone). Three rules share one kernel:
//   gated linear attention   S <- diag(a) S + k v^T;                                   o = S^T q
//   gated delta rule         S <- diag(a) S;  u = beta (v - S^T k);  S <- S + k u^T;   o = S^T q
//   read-out before the write, with a bonus for the current token
//                            o = S^T q + b v;  S <- diag(a) S + k v^T                  (b per token and head, given)
// with a decay per key channel a, given per token, head and channel (the product that makes its pre-activation z turns it
// into exp(-coef[head] * softplus(sign * z)); sign -1, coef 1 / tau gives sigmoid(z)^(1 / tau)). State, decays, gates and
// all sums are 32-bit. The columns of S are
// independent of one another, so a block owns a few columns of one (request, head) and walks the request's tokens in
// order; a column's rows are spread over KS lanes of a warp that add up with a fixed butterfly. What a token's result is
// does not depend on the batch or on how the tokens were cut into steps.
// Also here: the short causal convolution + SiLU + unit norm in front of the delta rule, the hand-over of the
// convolution's last inputs to the state slot, and the per-head RMS norm with an output gate behind both rules.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int WARPS = 4;
constexpr int RKMAX = 16;          // rows of a column that one lane holds
constexpr int MAX_TAPS = 16;
constexpr int SCAN_SMEM_BYTES = 40 * 1024;
constexpr int SCAN_VEC_ROWS = 16;
constexpr int SCAN_SPLIT_MIN = 256;  // tokens of a request in one step from which its portion is cut into parts that run side by side  // rows a lane holds in the kernel with 16-byte fetches, where the key size allows

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" :: "r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async16(float* smem, const float* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }

// The tokens of a request pass through shared memory in chunks of `chunk` tokens, two buffers taking turns: while the
// warps walk one chunk, the next one's q, k, z, v and beta are on their way (cp.async); when it has arrived the block
// squashes beta in place, once for all its columns.
template <int RULE>
__global__ void __launch_bounds__(WARPS * 32)
recurrent_scan_kernel(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* z, int ldz,
                      const float* beta, int ldb, float q_scale,
                      float* state, size_t slot_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                      float* out, int H, int G, int dk, int dv, int KS, int chunk, int vec) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr bool DELTA = RULE == BL_RULE_DELTA, BONUS = RULE == BL_RULE_BONUS;
    const int r = blockIdx.z, h = blockIdx.y;
    const int t0 = cu_q[r], n = cu_q[r + 1] - t0;
    if (n <= 0) return;
    const int gh = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int CW = 32 / KS, cols_blk = WARPS * CW;
    const int s = lane / CW, cc = lane % CW;
    const int c = (blockIdx.x * WARPS + warp) * CW + cc;
    const bool col_ok = c < dv;
    const int per_tok = 3 * dk + cols_blk + 4;              // q | k | decay | v | beta (+ padding to 16 bytes)
    const int buf_floats = chunk * per_tok;
    float* S = state + (size_t)slots[r] * slot_stride + (size_t)h * dk * dv;
    const int col0 = blockIdx.x * cols_blk;

    auto issue = [&](int base, float* buf) {
        const int m = min(chunk, n - base);
        for (int tt = warp; tt < m; tt += WARPS) {
            const size_t tok = (size_t)(t0 + base + tt);
            float* dst = buf + (size_t)tt * per_tok;
            const float* gq = q + tok * ldq + gh * dk;
            const float* gk = k + tok * ldk + gh * dk;
            const float* gz = z + tok * ldz + h * dk;
            if (vec) {
                for (int d = lane * 4; d < dk; d += 128) {
                    cp_async16(dst + d, gq + d); cp_async16(dst + dk + d, gk + d); cp_async16(dst + 2 * dk + d, gz + d);
                }
            } else {
                for (int d = lane; d < dk; d += 32) {
                    cp_async4(dst + d, gq + d); cp_async4(dst + dk + d, gk + d); cp_async4(dst + 2 * dk + d, gz + d);
                }
            }
            const float* gv = v + tok * ldv + h * dv + col0;
            for (int j = lane; j < cols_blk; j += 32) {
                if (col0 + j < dv) cp_async4(dst + 3 * dk + j, gv + j);
                else dst[3 * dk + j] = 0.f;
            }
            if ((DELTA || BONUS) && lane == 0) cp_async4(dst + 3 * dk + cols_blk, beta + tok * ldb + h);
        }
        cp_async_commit();
    };

    issue(0, sm);
    float st[RKMAX];
#pragma unroll
    for (int i = 0; i < RKMAX; ++i) {
        const int row = i * KS + s;
        st[i] = (row < dk && col_ok) ? S[(size_t)row * dv + c] : 0.f;
    }
    int which = 0;
    for (int base = 0; base < n; base += chunk, which ^= 1) {
        const int m = min(chunk, n - base);
        float* buf = sm + (size_t)which * buf_floats;
        if (base + chunk < n) { issue(base + chunk, sm + (size_t)(which ^ 1) * buf_floats); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        if (DELTA) {
            for (int tt = threadIdx.x; tt < m; tt += WARPS * 32) {
                float* b = buf + (size_t)tt * per_tok + 3 * dk + cols_blk;
                *b = sigmoidf_(*b);
            }
            __syncthreads();
        }
        // A token's q, k and decays are fetched into registers while the token before is worked on: the fetches do not
        // depend on the state, the arithmetic does, and a warp has no other warp to hide its latencies behind.
        float cq[RKMAX], ck[RKMAX], cd[RKMAX], nq[RKMAX], nk[RKMAX], nd[RKMAX];
        float cv, cb = 0.f, nv = 0.f, nb = 0.f;
        auto fetch = [&](int tt, float (&fq)[RKMAX], float (&fk)[RKMAX], float (&fd)[RKMAX], float& fv, float& fb) {
            const float* pq = buf + (size_t)tt * per_tok;
#pragma unroll
            for (int i = 0; i < RKMAX; ++i) {
                const int row = i * KS + s;
                const int rr = min(row, dk - 1);
                const bool ok = row < dk;
                fq[i] = ok ? pq[rr] : 0.f;
                fk[i] = ok ? pq[dk + rr] : 0.f;
                fd[i] = pq[2 * dk + rr];
            }
            fv = pq[3 * dk + warp * CW + cc];
            if (DELTA || BONUS) fb = pq[3 * dk + cols_blk];
        };
        fetch(0, cq, ck, cd, cv, cb);
        for (int tt = 0; tt < m; ++tt) {
            if (tt + 1 < m) fetch(tt + 1, nq, nk, nd, nv, nb);
            float o;
            if (!DELTA) {
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int i = 0; i < RKMAX; i += 2) {
                    if (BONUS) { o0 = fmaf(st[i], cq[i], o0); o1 = fmaf(st[i + 1], cq[i + 1], o1); }   // the state before the write
                    st[i] = fmaf(cd[i], st[i], ck[i] * cv);
                    st[i + 1] = fmaf(cd[i + 1], st[i + 1], ck[i + 1] * cv);
                    if (!BONUS) { o0 = fmaf(st[i], cq[i], o0); o1 = fmaf(st[i + 1], cq[i + 1], o1); }
                }
                o = o0 + o1;
                for (int x = 16; x >= CW; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
                if (BONUS) o = fmaf(cb, cv, o);
            } else {
                float sk0 = 0.f, sk1 = 0.f, sq0 = 0.f, sq1 = 0.f, kq0 = 0.f, kq1 = 0.f;
#pragma unroll
                for (int i = 0; i < RKMAX; i += 2) {
                    st[i] *= cd[i];
                    st[i + 1] *= cd[i + 1];
                    sk0 = fmaf(st[i], ck[i], sk0); sk1 = fmaf(st[i + 1], ck[i + 1], sk1);
                    sq0 = fmaf(st[i], cq[i], sq0); sq1 = fmaf(st[i + 1], cq[i + 1], sq1);
                    kq0 = fmaf(ck[i], cq[i], kq0); kq1 = fmaf(ck[i + 1], cq[i + 1], kq1);
                }
                float sk_ = sk0 + sk1, sq_ = sq0 + sq1, kq = kq0 + kq1;
                for (int x = 16; x >= CW; x >>= 1) {
                    sk_ += __shfl_xor_sync(0xffffffffu, sk_, x);
                    sq_ += __shfl_xor_sync(0xffffffffu, sq_, x);
                    kq += __shfl_xor_sync(0xffffffffu, kq, x);
                }
                const float u = cb * (cv - sk_);
#pragma unroll
                for (int i = 0; i < RKMAX; ++i) st[i] = fmaf(ck[i], u, st[i]);
                o = fmaf(kq, u, sq_);                  // S^T q after the write: (a S)^T q + (k . q) u
            }
            if (s == 0 && col_ok) out[(size_t)(t0 + base + tt) * H * dv + h * dv + c] = o * q_scale;
#pragma unroll
            for (int i = 0; i < RKMAX; ++i) { cq[i] = nq[i]; ck[i] = nk[i]; cd[i] = nd[i]; }
            cv = nv; cb = nb;
        }
        __syncthreads();                               // the buffer is free for the chunk after next
    }
#pragma unroll
    for (int i = 0; i < RKMAX; ++i) {
        const int row = i * KS + s;
        if (row < dk && col_ok) S[(size_t)row * dv + c] = st[i];
    }
}

// The same walk for key sizes that split evenly: a lane holds RK4 * 4 CONSECUTIVE rows of its column (dk = KS * RK4 * 4),
// so a token's q, k and decays reach its registers as 16-byte loads at fixed offsets, two tokens' registers take turns
// (no copies), and the dot products run in two chains. A warp has no other warp on its scheduler to hide latencies
// behind (a request gives H * dv / (WARPS * CW) blocks): what counts is the number of instructions per token.
template <int RULE, int RK4>
__global__ void __launch_bounds__(WARPS * 32)
recurrent_scan_vec_kernel(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* z, int ldz,
                          const float* beta, int ldb, float q_scale,
                          float* state, size_t slot_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                          float* out, int H, int G, int dk, int dv, int KS, int chunk, int vec,
                          int nc, int pass, float* part_s, float* part_p, const float* part_start) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr bool DELTA = RULE == BL_RULE_DELTA, BONUS = RULE == BL_RULE_BONUS;
    constexpr int RK = RK4 * 4;
    // A long portion of a request may be cut into nc parts that run side by side (linear attention only: its recurrence is
    // linear in S with a diagonal transition). pass 1: every part from a ZERO state, leaving its own contribution S_part and
    // the product P of its decays; pass 2: a part starts from the request's state folded through the parts before it
    // (S <- P o S + S_part) and writes the outputs; a small kernel then folds all parts into the slot. The delta rule's
    // transition is a matrix: its fold (S <- P S + S_part, a small product) runs between the passes, leaves every part's
    // start state in scratch and the final state in the slot. Short portions
    // (and nc 1) take one block per (request, head, columns) through pass 0 / 2 as before.
    const int r = blockIdx.z / nc, part = blockIdx.z % nc, h = blockIdx.y;
    const int n_all = cu_q[r + 1] - cu_q[r];
    if (n_all <= 0) return;
    const bool split = nc > 1 && n_all >= SCAN_SPLIT_MIN;
    if (!split && (part != 0 || pass == 1)) return;
    const int part_len = split ? (n_all + nc - 1) / nc : n_all;
    const int t_first = split ? part * part_len : 0;
    const int t0 = cu_q[r] + t_first, n = min(n_all - t_first, part_len);
    if (n <= 0) return;
    const int gh = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int CW = 32 / KS, cols_blk = WARPS * CW;
    const int s = lane / CW, cc = lane % CW;
    const int c = (blockIdx.x * WARPS + warp) * CW + cc;
    // The delta rule's transition over a part is a key x key matrix: pass 1 makes it in dk further columns that start as
    // the identity and see values of zero (column dv + j ends as the part's transition applied to unit vector j).
    const int n_cols = dv + (DELTA && split && pass == 1 ? dk : 0);
    const bool col_ok = c < n_cols;
    const int per_tok = 3 * dk + cols_blk + 4;
    const int buf_floats = chunk * per_tok;
    float* S = state + (size_t)slots[r] * slot_stride + (size_t)h * dk * dv;
    const int col0 = blockIdx.x * cols_blk;
    if (col0 >= n_cols) return;
    const int row0 = s * RK;

    auto issue = [&](int base, float* buf) {
        const int m = min(chunk, n - base);
        for (int tt = warp; tt < m; tt += WARPS) {
            const size_t tok = (size_t)(t0 + base + tt);
            float* dst = buf + (size_t)tt * per_tok;
            const float* gq = q + tok * ldq + gh * dk;
            const float* gk = k + tok * ldk + gh * dk;
            const float* gz = z + tok * ldz + h * dk;
            if (vec) {
                for (int d = lane * 4; d < dk; d += 128) {
                    cp_async16(dst + d, gq + d); cp_async16(dst + dk + d, gk + d); cp_async16(dst + 2 * dk + d, gz + d);
                }
            } else {
                for (int d = lane; d < dk; d += 32) {
                    cp_async4(dst + d, gq + d); cp_async4(dst + dk + d, gk + d); cp_async4(dst + 2 * dk + d, gz + d);
                }
            }
            const float* gv = v + tok * ldv + h * dv + col0;
            for (int j = lane; j < cols_blk; j += 32) {
                if (col0 + j < dv) cp_async4(dst + 3 * dk + j, gv + j);
                else dst[3 * dk + j] = 0.f;
            }
            if ((DELTA || BONUS) && lane == 0) cp_async4(dst + 3 * dk + cols_blk, beta + tok * ldb + h);
        }
        cp_async_commit();
    };

    issue(0, sm);
    float st[RK], pr[RK];
    const size_t part_base = ((size_t)r * nc) * H + h;           // + p * H for part p
#pragma unroll
    for (int i = 0; i < RK; ++i) {
        if (split && pass == 1) st[i] = (DELTA && c >= dv && row0 + i == c - dv) ? 1.f : 0.f;
        else if (DELTA && split) st[i] = col_ok ? part_start[((part_base + (size_t)part * H) * dk + row0 + i) * dv + c] : 0.f;
        else st[i] = col_ok ? S[(size_t)(row0 + i) * dv + c] : 0.f;
        pr[i] = 1.f;
    }
    if (!DELTA && split && pass == 2) {
        for (int p = 0; p < part; ++p) {
            const float* ps = part_s + (part_base + (size_t)p * H) * dk * dv;
            const float* pp = part_p + (part_base + (size_t)p * H) * dk;
#pragma unroll
            for (int i = 0; i < RK; ++i)
                st[i] = col_ok ? fmaf(pp[row0 + i], st[i], ps[(size_t)(row0 + i) * dv + c]) : 0.f;
        }
    }
    const bool quiet = split && pass == 1;                       // no outputs yet
    const int v_off = 3 * dk + warp * CW + cc, b_off = 3 * dk + cols_blk;
    const int dk4 = dk >> 2;

    struct Tok { float4 q[RK4], k[RK4], d[RK4]; float v, b; };
    auto fetch = [&](const float* tokp, Tok& t) {
        const float4* p4 = reinterpret_cast<const float4*>(tokp + row0);
#pragma unroll
        for (int j = 0; j < RK4; ++j) { t.q[j] = p4[j]; t.k[j] = p4[dk4 + j]; t.d[j] = p4[2 * dk4 + j]; }
        t.v = tokp[v_off];
        t.b = (DELTA || BONUS) ? tokp[b_off] : 0.f;
    };
    auto step = [&](const Tok& t, size_t tok) {
        const float* tq = reinterpret_cast<const float*>(t.q);
        const float* tk = reinterpret_cast<const float*>(t.k);
        const float* td = reinterpret_cast<const float*>(t.d);
        float o;
        if (!DELTA) {
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < RK; i += 2) {
                if (BONUS) { o0 = fmaf(st[i], tq[i], o0); o1 = fmaf(st[i + 1], tq[i + 1], o1); }       // the state before the write
                st[i] = fmaf(td[i], st[i], tk[i] * t.v);
                st[i + 1] = fmaf(td[i + 1], st[i + 1], tk[i + 1] * t.v);
                if (!BONUS) { o0 = fmaf(st[i], tq[i], o0); o1 = fmaf(st[i + 1], tq[i + 1], o1); }
            }
            if (quiet) {
#pragma unroll
                for (int i = 0; i < RK; ++i) pr[i] *= td[i];
                return;
            }
            o = o0 + o1;
            for (int x = 16; x >= CW; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (BONUS) o = fmaf(t.b, t.v, o);
        } else {
            float sk0 = 0.f, sk1 = 0.f, sq0 = 0.f, sq1 = 0.f, kq0 = 0.f, kq1 = 0.f;
#pragma unroll
            for (int i = 0; i < RK; i += 2) {
                st[i] *= td[i];
                st[i + 1] *= td[i + 1];
                sk0 = fmaf(st[i], tk[i], sk0); sk1 = fmaf(st[i + 1], tk[i + 1], sk1);
                sq0 = fmaf(st[i], tq[i], sq0); sq1 = fmaf(st[i + 1], tq[i + 1], sq1);
                kq0 = fmaf(tk[i], tq[i], kq0); kq1 = fmaf(tk[i + 1], tq[i + 1], kq1);
            }
            float sk_ = sk0 + sk1, sq_ = sq0 + sq1, kq = kq0 + kq1;
            for (int x = 16; x >= CW; x >>= 1) {
                sk_ += __shfl_xor_sync(0xffffffffu, sk_, x);
                sq_ += __shfl_xor_sync(0xffffffffu, sq_, x);
                kq += __shfl_xor_sync(0xffffffffu, kq, x);
            }
            const float u = t.b * (t.v - sk_);
#pragma unroll
            for (int i = 0; i < RK; ++i) st[i] = fmaf(tk[i], u, st[i]);
            o = fmaf(kq, u, sq_);
        }
        if (s == 0 && col_ok && !quiet) out[tok * H * dv + h * dv + c] = o * q_scale;
    };

    int which = 0;
    for (int base = 0; base < n; base += chunk, which ^= 1) {
        const int m = min(chunk, n - base);
        float* buf = sm + (size_t)which * buf_floats;
        if (base + chunk < n) { issue(base + chunk, sm + (size_t)(which ^ 1) * buf_floats); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        if (DELTA) {
            for (int tt = threadIdx.x; tt < m; tt += WARPS * 32) {
                float* b = buf + (size_t)tt * per_tok + b_off;
                *b = sigmoidf_(*b);
            }
            __syncthreads();
        }
        Tok ta, tb;
        fetch(buf, ta);
        const size_t tok0 = (size_t)(t0 + base);
        int tt = 0;
        for (; tt + 1 < m; tt += 2) {
            fetch(buf + (size_t)(tt + 1) * per_tok, tb);
            step(ta, tok0 + tt);
            if (tt + 2 < m) fetch(buf + (size_t)(tt + 2) * per_tok, ta);
            step(tb, tok0 + tt + 1);
        }
        if (tt < m) step(ta, tok0 + tt);
        __syncthreads();                               // the buffer is free for the chunk after next
    }
    if (split) {
        if (pass == 1 && DELTA) {
            float* ps = part_s + (part_base + (size_t)part * H) * dk * dv;
            float* pm = part_p + (part_base + (size_t)part * H) * dk * dk;      // [row][unit vector]
#pragma unroll
            for (int i = 0; i < RK; ++i) {
                if (c < dv) ps[(size_t)(row0 + i) * dv + c] = st[i];
                else if (col_ok) pm[(size_t)(row0 + i) * dk + (c - dv)] = st[i];
            }
        } else if (pass == 1) {
            float* ps = part_s + (part_base + (size_t)part * H) * dk * dv;
            float* pp = part_p + (part_base + (size_t)part * H) * dk;
#pragma unroll
            for (int i = 0; i < RK; ++i) {
                if (col_ok) ps[(size_t)(row0 + i) * dv + c] = st[i];
                if (blockIdx.x == 0 && warp == 0 && cc == 0) pp[row0 + i] = pr[i];
            }
        }
        return;                                        // the slot is written by the fold behind pass 2
    }
#pragma unroll
    for (int i = 0; i < RK; ++i)
        if (col_ok) S[(size_t)(row0 + i) * dv + c] = st[i];
}

// Between the two passes of a cut portion of the delta rule: start[0] = the slot's state, start[p + 1] = P_p start[p] +
// S_part_p (P_p a key x key matrix), the last one into the slot. A block owns FOLD_COLS columns of one (request, head) and
// keeps the current state's columns in shared memory, two buffers taking turns.
constexpr int FOLD_COLS = 32, FOLD_MAX_DK = 128;
__global__ void __launch_bounds__(256)
scan_fold_matrix_kernel(float* state, size_t slot_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                        const float* part_s, const float* part_pm, float* part_start, int H, int dk, int dv, int nc) {
    bl_pdl_trigger();
    bl_pdl_wait();
    __shared__ float cur[2][FOLD_MAX_DK][FOLD_COLS];
    const int r = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * FOLD_COLS;
    if (cu_q[r + 1] - cu_q[r] < SCAN_SPLIT_MIN) return;
    float* S = state + (size_t)slots[r] * slot_stride + (size_t)h * dk * dv;
    const size_t base = ((size_t)r * nc) * H + h;
    const int col = threadIdx.x % FOLD_COLS, rg = threadIdx.x / FOLD_COLS;      // 8 row groups
    const bool ok = c0 + col < dv;
    for (int row = rg; row < dk; row += 8) {
        const float x = ok ? S[(size_t)row * dv + c0 + col] : 0.f;
        cur[0][row][col] = x;
        if (ok) part_start[((base + 0) * dk + row) * dv + c0 + col] = x;
    }
    __syncthreads();
    int w = 0;
    for (int p = 0; p < nc; ++p, w ^= 1) {
        const float* pm = part_pm + (base + (size_t)p * H) * dk * dk;
        const float* ps = part_s + (base + (size_t)p * H) * dk * dv;
        for (int row = rg; row < dk; row += 8) {
            float acc = ok ? ps[(size_t)row * dv + c0 + col] : 0.f;
            const float* prow = pm + (size_t)row * dk;
            for (int j = 0; j < dk; ++j) acc = fmaf(prow[j], cur[w][j][col], acc);
            cur[w ^ 1][row][col] = acc;
            if (ok) {
                if (p + 1 < nc) part_start[((base + (size_t)(p + 1) * H) * dk + row) * dv + c0 + col] = acc;
                else S[(size_t)row * dv + c0 + col] = acc;
            }
        }
        __syncthreads();
    }
}

// Behind the two passes of a cut portion: the request's state folded through all parts, into its slot.
__global__ void scan_fold_kernel(float* state, size_t slot_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                                 const float* part_s, const float* part_p, int H, int dk, int dv, int nc) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int r = blockIdx.z, h = blockIdx.y;
    if (cu_q[r + 1] - cu_q[r] < SCAN_SPLIT_MIN) return;
    float* S = state + (size_t)slots[r] * slot_stride + (size_t)h * dk * dv;
    const size_t base = ((size_t)r * nc) * H + h;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= dk * dv) return;
    const int row = e / dv;
    float sv = S[e];
#pragma unroll 4
    for (int p = 0; p < nc; ++p)
        sv = fmaf(part_p[(base + (size_t)p * H) * dk + row], sv, part_s[(base + (size_t)p * H) * dk * dv + e]);
    S[e] = sv;
}

// y[t, h, :] = u / sqrt(mean(u^2) + eps) * w * gate(g[t, h, :]); w is one vector of dv values shared by the heads, or
// (w_per_head) H * dv values. The heads of a row of o lie o_head_stride values apart. floor null: u = o[t, h, :dv]; else
// u = o[t, h, :dv] / (max(|o[t, h, dv]|, floor[t, h]) + 1e-6): the read-out of a matrix memory whose normaliser was walked
// as one more value column. One warp per (token, head).
template <typename TY>
__global__ void __launch_bounds__(WARPS * 32)
head_norm_gate_kernel(const float* o, int o_head_stride, const void* __restrict__ w, int w_dtype, int w_per_head, const float* floor,
                      const float* gate, int ld_gate, int gate_kind, TY* __restrict__ y, int items, int H, int dv, float eps) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (item >= items) return;
    const int t = item / H, h = item % H;
    const float* src = o + (size_t)item * o_head_stride;
    const float pre = floor ? 1.0f / (fmaxf(fabsf(src[dv]), floor[item]) + 1e-6f) : 1.0f;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) { const float u = src[i] * pre; ss += u * u; }
    const float inv = pre / sqrtf(bl_warp_sum(ss) / (float)dv + eps);
    const float* g = gate ? gate + (size_t)t * ld_gate + h * dv : nullptr;
    const size_t w0 = w_per_head ? (size_t)h * dv : 0;
    for (int i = lane; i < dv; i += 32) {
        float val = src[i] * inv * (w ? bl_load_any(w, w_dtype, w0 + i) : 1.f);
        if (g) val *= gate_kind == BL_GATE_SILU ? bl_silu(g[i]) : sigmoidf_(g[i]);
        bl_store(y + (size_t)item * dv + i, val);
    }
}

// The gates of a matrix memory with exponential gating: one warp per (request, head) walks the request's tokens in order.
// Per token: log input gate i = cap tanh((zi + bi) / cap), log forget gate f = log sigmoid(cap tanh((zf + bf) / cap)), the
// running maximum m' = max(f + m, i) (m starts at 0 in a fresh slot and is kept in the slot at off_m), and from them the
// decay a = e^(f + m - m'), the input weight e = e^(i - m') and the floor e^(-m') of the read-out's denominator, into
// gates [3, T, H]. 32 tokens at a time: their gates in parallel (a lane each; the next 32 tokens' pre-activations are
// fetched before), the maxima as a chain of 32 steps of two dependent instructions.
__global__ void __launch_bounds__(32)
memory_gate_chain_kernel(const float* proj, int ld, int off_i, int off_f, const void* __restrict__ bi, int bi_dtype,
                         const void* __restrict__ bf, int bf_dtype, float cap, float* state, size_t slot_stride, size_t off_m,
                         const int* __restrict__ slots, const int* __restrict__ cu_q, float* gates, int T, int H) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int r = blockIdx.y, h = blockIdx.x, lane = threadIdx.x;
    const int t0 = cu_q[r], n_tok = cu_q[r + 1] - t0;
    if (n_tok <= 0) return;
    float* mp = state + (size_t)slots[r] * slot_stride + off_m + h;
    float m = *mp;
    const float b_i = bl_load_any(bi, bi_dtype, h), b_f = bl_load_any(bf, bf_dtype, h);
    const float inv_cap = 1.0f / cap;
    float zi = 0.f, zf = 0.f;
    if (lane < n_tok) { const float* row = proj + (size_t)(t0 + lane) * ld; zi = row[off_i + h]; zf = row[off_f + h]; }
    for (int base = 0; base < n_tok; base += 32) {
        const int cnt = min(32, n_tok - base);
        float nzi = 0.f, nzf = 0.f;
        if (base + 32 + lane < n_tok) { const float* row = proj + (size_t)(t0 + base + 32 + lane) * ld; nzi = row[off_i + h]; nzf = row[off_f + h]; }
        const float gi = cap * tanhf((zi + b_i) * inv_cap);
        const float z = cap * tanhf((zf + b_f) * inv_cap);
        const float gf = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
        float m_before = 0.f, m_mine = 0.f;
        for (int tt = 0; tt < cnt; ++tt) {
            const float f_t = __shfl_sync(0xffffffffu, gf, tt), i_t = __shfl_sync(0xffffffffu, gi, tt);
            const float m_new = fmaxf(f_t + m, i_t);
            if (lane == tt) { m_before = m; m_mine = m_new; }
            m = m_new;
        }
        if (lane < cnt) {
            const size_t at = (size_t)(t0 + base + lane) * H + h;
            gates[at] = expf(gf + m_before - m_mine);
            gates[(size_t)T * H + at] = expf(gi - m_mine);
            gates[2 * (size_t)T * H + at] = expf(-m_mine);
        }
        zi = nzi; zf = nzf;
    }
    if (lane == 0) *mp = m;
}

// What the scan of a matrix memory reads, from the projections and the gates: decay[t, h, :] = a[t, h] for every key
// channel, k_out[t, h, :] = e[t, h] * k[t, h, :], v_out[t, h, :] = (v[t, h, :], 1): the one in the last column makes the
// normaliser n the state's last value column, and n . q the last column of the read-out. One block per token.
__global__ void __launch_bounds__(WARPS * 32)
memory_expand_kernel(const float* proj, int ld, int off_k, int off_v, const float* __restrict__ gates, float* decay, float* k_out,
                     float* v_out, int T, int H, int dk, int dv) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    for (int e = threadIdx.x; e < H * dk; e += WARPS * 32) {
        const size_t g = (size_t)t * H + e / dk;
        decay[(size_t)t * H * dk + e] = gates[g];
        k_out[(size_t)t * H * dk + e] = gates[(size_t)T * H + g] * row[off_k + e];
    }
    for (int e = threadIdx.x; e < H * (dv + 1); e += WARPS * 32) {
        const int h = e / (dv + 1), c = e % (dv + 1);
        v_out[(size_t)t * H * (dv + 1) + e] = c < dv ? row[off_v + h * dv + c] : 1.0f;
    }
}

// Token shift: out[s, t, c] = x[t, c] + (x'[t, c] - x[t, c]) * mu[s, c] for s < n_mix, x' the row of the request's token
// before (from the slot's `prev` [d] for a step's first token: zeros in a fresh slot). One block per token; four channels
// a thread (16-byte loads, 8- or 16-byte stores) where the rows allow it.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 pk;
    pk.x = *reinterpret_cast<const unsigned*>(&lo); pk.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = pk;
}

template <typename TY>
__global__ void __launch_bounds__(WARPS * 32)
shift_mix_kernel(const float* x, int ld, const float* __restrict__ mu, int n_mix, const float* prev, size_t slot_stride,
                 const int* __restrict__ slots, const int* __restrict__ tok_req, const int* __restrict__ cu_q, TY* __restrict__ out,
                 int T, int d, int vec) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int t = blockIdx.x;
    const int r = tok_req[t];
    const float* before = t > cu_q[r] ? x + (size_t)(t - 1) * ld : prev + (size_t)slots[r] * slot_stride;
    const float* cur = x + (size_t)t * ld;
    if (vec) {
        for (int c = threadIdx.x * 4; c < d; c += WARPS * 32 * 4) {
            const float4 xc = *reinterpret_cast<const float4*>(cur + c), xb = *reinterpret_cast<const float4*>(before + c);
            const float4 dx = make_float4(xb.x - xc.x, xb.y - xc.y, xb.z - xc.z, xb.w - xc.w);
            for (int s = 0; s < n_mix; ++s) {
                const float4 m = *reinterpret_cast<const float4*>(mu + (size_t)s * d + c);
                store4(out + ((size_t)s * T + t) * d + c, fmaf(dx.x, m.x, xc.x), fmaf(dx.y, m.y, xc.y), fmaf(dx.z, m.z, xc.z), fmaf(dx.w, m.w, xc.w));
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < d; c += WARPS * 32) {
        const float xc = cur[c], dx = before[c] - xc;
        for (int s = 0; s < n_mix; ++s)
            bl_store(out + ((size_t)s * T + t) * d + c, fmaf(dx, mu[(size_t)s * d + c], xc));
    }
}

// b[t, h] = sum_c u[h, c] * k[t, h, c] * q[t, h, c]: what the current token adds to its own read-out; one warp per (t, h).
__global__ void __launch_bounds__(WARPS * 32)
bonus_dot_kernel(const float* q, int ldq, const float* k, int ldk, const void* __restrict__ u, int u_dtype, float* out,
                 int items, int H, int dk) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (item >= items) return;
    const int t = item / H, h = item % H;
    const float* qr = q + (size_t)t * ldq + (size_t)h * dk;
    const float* kr = k + (size_t)t * ldk + (size_t)h * dk;
    float acc = 0.f;
    for (int c = lane; c < dk; c += 32) acc = fmaf(bl_load_any(u, u_dtype, (size_t)h * dk + c) * kr[c], qr[c], acc);
    acc = bl_warp_sum(acc);
    if (lane == 0) out[item] = acc;
}

// One block per token: y[t, ch] = silu(sum_i taps[ch, i] * x[t - (n_taps - 1) + i, ch]), the inputs before the step's
// first token of the request coming from the slot's tail (its last n_taps - 1 inputs, oldest first; zeros at the
// start of a sequence). Then the first `unit_heads` heads of `dk` columns are made unit vectors, x / sqrt(sum x^2 +
// unit_eps), the first `scaled_heads` of them also times q_scale.
__global__ void __launch_bounds__(WARPS * 32)
conv_silu_unit_kernel(const float* x, int ld, const float* __restrict__ taps, int n_taps, const float* tail, size_t slot_stride,
                      const int* __restrict__ slots, const int* __restrict__ tok_req, const int* __restrict__ cu_q, float* y,
                      int C, int unit_heads, int scaled_heads, int dk, float q_scale, float unit_eps, const void* __restrict__ bias,
                      int bias_dtype) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int t = blockIdx.x;
    const int r = tok_req[t];
    const int j = t - cu_q[r];
    const float* tl = tail + (size_t)slots[r] * slot_stride;
    for (int ch = threadIdx.x; ch < C; ch += WARPS * 32) {
        float acc = bias ? bl_load_any(bias, bias_dtype, ch) : 0.f;
        for (int i = 0; i < n_taps; ++i) {
            const int off = j - (n_taps - 1) + i;
            const float xv = off >= 0 ? x[(size_t)(t - j + off) * ld + ch] : tl[(size_t)(n_taps - 1 + off) * C + ch];
            acc = fmaf(taps[(size_t)ch * n_taps + i], xv, acc);
        }
        y[(size_t)t * C + ch] = bl_silu(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    for (int hh = threadIdx.x >> 5; hh < unit_heads; hh += WARPS) {
        float* p = y + (size_t)t * C + (size_t)hh * dk;
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss += p[d] * p[d];
        const float inv = (hh < scaled_heads ? q_scale : 1.f) / sqrtf(bl_warp_sum(ss) + unit_eps);
        for (int d = lane; d < dk; d += 32) p[d] *= inv;
    }
}

// After the step's convolutions have read the tail: the last n_taps - 1 inputs of each request with tokens.
__global__ void conv_tail_update_kernel(const float* x, int ld, int n_taps, float* tail, size_t slot_stride,
                                        const int* __restrict__ slots, const int* __restrict__ cu_q, int C) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int r = blockIdx.y;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = cu_q[r], n = cu_q[r + 1] - t0;
    if (n <= 0 || ch >= C) return;
    float* tl = tail + (size_t)slots[r] * slot_stride;
    float keep[MAX_TAPS];
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i) {
        if (i < n_taps - 1) {
            const int off = n - (n_taps - 1) + i;
            keep[i] = off >= 0 ? x[(size_t)(t0 + off) * ld + ch] : tl[(size_t)(n_taps - 1 + off) * C + ch];
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i)
        if (i < n_taps - 1) tl[(size_t)i * C + ch] = keep[i];
}


// In front of a recurrence with a FIXED decay per head (retention): q and k of every head rotated by the token's position
// (the first 2 * rot_half values of a head in pairs (i, i + rot_half), angle = float(position) * inv_freq[i], all 32-bit),
// k times k_scale after the rotation, and the head's decay written for each of its key channels (what the scan reads).
// One block per token.
__global__ void __launch_bounds__(WARPS * 32)
rope_decay_prep_kernel(const float* proj, int ld, int off_k, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                       int rot_half, const float* __restrict__ head_decay, float k_scale, float* q_out, float* k_out,
                       float* decay_out, int H, int dk) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    const float* src = proj + (size_t)t * ld;
    const size_t row = (size_t)t * H * dk;
    for (int e = threadIdx.x; e < H * dk; e += WARPS * 32) {
        const int h = e / dk, d = e % dk;
        float qv = src[e], kv = src[off_k + e];
        if (d < 2 * rot_half) {
            const int i = d < rot_half ? d : d - rot_half;
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            const int other = d < rot_half ? e + rot_half : e - rot_half;
            const float qo = src[other], ko = src[off_k + other];
            if (d < rot_half) { qv = qv * cs - qo * sn; kv = kv * cs - ko * sn; }
            else { qv = qv * cs + qo * sn; kv = kv * cs + ko * sn; }
        }
        q_out[row + e] = qv;
        k_out[row + e] = kv * k_scale;
        decay_out[row + e] = head_decay[h];
    }
}

// In front of a selective state-space recurrence (one decay per head and token): dt = softplus(raw + dt_bias[h]);
// decay[t, h, :] = exp(-exp(A_log[h]) * dt) for each of the n_state key channels; v[t, h, :] = dt * x[t, h, :].
// raw: 32-bit rows [T, >= H]; x: [T, H * dv] (the convolved inputs). neg_rate[h] = exp(A_log[h]), made at load. One block per token.
__global__ void __launch_bounds__(WARPS * 32)
ssd_prep_kernel(const float* raw, int ld_raw, const void* __restrict__ dt_bias, int bias_dtype, const float* __restrict__ rate,
                const float* x, int ld_x, float* decay_out, float* v_out, int H, int n_state, int dv) {
    bl_pdl_trigger();
    bl_pdl_wait();
    __shared__ float dts[256];
    const int t = blockIdx.x;
    for (int h0 = 0; h0 < H; h0 += 256) {
        const int hn = min(256, H - h0);
        __syncthreads();
        for (int h = threadIdx.x; h < hn; h += WARPS * 32) {
            const float zz = raw[(size_t)t * ld_raw + h0 + h] + bl_load_any(dt_bias, bias_dtype, h0 + h);
            dts[h] = zz > 20.f ? zz : log1pf(expf(zz));
        }
        __syncthreads();
        for (int e = threadIdx.x; e < hn * n_state; e += WARPS * 32) {
            const int h = e / n_state;
            decay_out[((size_t)t * H + h0) * n_state + e] = expf(-rate[h0 + h] * dts[h]);
        }
        for (int e = threadIdx.x; e < hn * dv; e += WARPS * 32) {
            const int h = e / dv;
            v_out[((size_t)t * H + h0) * dv + e] = dts[h] * x[(size_t)t * ld_x + (size_t)h0 * dv + e];
        }
    }
}

// Behind such a recurrence: u = (o + skip[h] * x) * silu(z) (the gate comes BEFORE the norm), then an RMS norm over each of
// n_parts equal parts of the row (each part by its own root mean square), times w. One block per (token, part); a part may
// span several heads or a fraction of one. skip and x may be null (no skip term), z may be null (no gate). A thread keeps
// up to GN_KEEP of its values between the two passes (parts of up to GN_KEEP * 128 values are read once); the sum of squares
// is added in a fixed order (lanes, then warps).
constexpr int GN_KEEP = 16;
template <typename TY>
__global__ void __launch_bounds__(WARPS * 32)
gated_group_norm_kernel(const float* o, const float* x, int ld_x, const void* __restrict__ skip, int skip_dtype, int dv,
                        const float* z, int ld_z, const void* __restrict__ w, int w_dtype, TY* __restrict__ y, int n_parts,
                        int width, float eps) {
    bl_pdl_trigger();
    bl_pdl_wait();
    __shared__ float warp_ss[WARPS];
    const int t = blockIdx.x / n_parts, part = blockIdx.x % n_parts;
    const int per = width / n_parts, c0 = part * per;
    auto value = [&](int c) {
        float u = o[(size_t)t * width + c];
        if (x) u = fmaf(bl_load_any(skip, skip_dtype, c / dv), x[(size_t)t * ld_x + c], u);
        if (z) u *= bl_silu(z[(size_t)t * ld_z + c]);
        return u;
    };
    float keep[GN_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < GN_KEEP; ++j) {
        const int i = threadIdx.x + j * WARPS * 32;
        keep[j] = i < per ? value(c0 + i) : 0.f;
        ss += keep[j] * keep[j];
    }
    for (int i = threadIdx.x + GN_KEEP * WARPS * 32; i < per; i += WARPS * 32) { const float u = value(c0 + i); ss += u * u; }
    ss = bl_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < WARPS; ++k) total += warp_ss[k];
    const float inv = 1.0f / sqrtf(total / (float)per + eps);
#pragma unroll
    for (int j = 0; j < GN_KEEP; ++j) {
        const int i = threadIdx.x + j * WARPS * 32;
        if (i < per) bl_store(y + (size_t)t * width + c0 + i, keep[j] * inv * (w ? bl_load_any(w, w_dtype, c0 + i) : 1.f));
    }
    for (int i = threadIdx.x + GN_KEEP * WARPS * 32; i < per; i += WARPS * 32)
        bl_store(y + (size_t)t * width + c0 + i, value(c0 + i) * inv * (w ? bl_load_any(w, w_dtype, c0 + i) : 1.f));
}

}  // namespace

extern "C" int bl_recurrent_scan(int rule, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                 const float* z, int ldz, const float* beta, int ldb, float q_scale, float* state, long long slot_stride, const int* slots, const int* cu_q, int R,
                                 float* out, int H, int G, int dk, int dv, void* stream) {
    return bl_recurrent_scan_parts(rule, q, ldq, k, ldk, v, ldv, z, ldz, beta, ldb, q_scale, state, slot_stride, slots, cu_q, R, out,
                                   H, G, dk, dv, 1, nullptr, stream);
}

// Whether bl_recurrent_scan_parts can cut long portions of this rule and key size (else it runs them in one piece):
// 0, or the blocks that each part of one request's portion runs on in the first pass, H * ceil(columns / columns a
// block) (the delta rule's first pass has dk columns more, and its fold takes key sizes up to 128).
extern "C" int bl_recurrent_scan_can_split(int rule, int H, int dk, int dv) {
    if (rule != BL_RULE_GLA && rule != BL_RULE_DELTA && rule != BL_RULE_BONUS) return 0;
    if (rule == BL_RULE_DELTA && dk > FOLD_MAX_DK) return 0;
    for (int ks = 1; ks <= 32; ks *= 2)
        if (dk % (4 * ks) == 0 && dk / ks <= SCAN_VEC_ROWS) {
            const int cols_blk = WARPS * (32 / ks), cols = dv + (rule == BL_RULE_DELTA ? dk : 0);
            return H * ((cols + cols_blk - 1) / cols_blk);
        }
    return 0;
}

// Floats of scratch that bl_recurrent_scan_parts needs.
extern "C" long long bl_recurrent_scan_parts_scratch(int rule, int R, int nc, int H, int dk, int dv) {
    const long long per = rule == BL_RULE_DELTA ? (long long)dk * (2 * dv + dk) : (long long)dk * (dv + 1);
    return (long long)R * nc * H * per;
}

extern "C" int bl_recurrent_scan_parts(int rule, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                       const float* z, int ldz, const float* beta, int ldb, float q_scale, float* state,
                                       long long slot_stride, const int* slots, const int* cu_q, int R, float* out, int H, int G,
                                       int dk, int dv, int nc, float* scratch, void* stream) {
    if (R <= 0) return 0;
    if (nc < 1 || (nc > 1 && (scratch == nullptr || !bl_recurrent_scan_can_split(rule, H, dk, dv) || (long long)R * nc > 65535)))
        BL_FAIL("bl_recurrent_scan_parts: %d parts for rule %d, %d key channels, %d requests", nc, rule, dk, R);
    if (H <= 0 || G <= 0 || H % G != 0 || dk <= 0 || dv <= 0) BL_FAIL("bl_recurrent_scan: bad sizes H=%d G=%d dk=%d dv=%d", H, G, dk, dv);
    if (dk > RKMAX * 32) BL_FAIL("bl_recurrent_scan: %d key channels, at most %d", dk, RKMAX * 32);
    if (R > 65535 || H > 65535) BL_FAIL("bl_recurrent_scan: %d requests or %d heads are too many for one launch", R, H);
    if ((rule == BL_RULE_DELTA || rule == BL_RULE_BONUS) && beta == nullptr) BL_FAIL("bl_recurrent_scan: rule %d needs beta", rule);
    int KS = 1;
    while ((dk + KS - 1) / KS > RKMAX) KS *= 2;
    // The kernel with 16-byte fetches where the key size splits evenly over the lanes. Sixteen rows a lane: eight, with a
    // butterfly of one more step, were measured and are no faster for one request (64 x 128 heads, 2,048 tokens: 534 us
    // against 570) and slower where it counts, 128 x 256 heads (752 against 678) and decode steps of 64 requests (115 us
    // against 67): a token's time is its chain of dependent instructions, not its arithmetic.
    int rk4 = 0;
    for (int ks = 1; ks <= 32 && rk4 == 0; ks *= 2)
        if (dk % (4 * ks) == 0 && dk / ks <= SCAN_VEC_ROWS) { KS = ks; rk4 = dk / (4 * ks); }
    if (rk4 == 0 && dk % (4 * KS) == 0) rk4 = dk / (4 * KS);
    const int CW = 32 / KS, cols_blk = WARPS * CW;
    const size_t per_token = (size_t)(3 * dk + cols_blk + 4) * sizeof(float);
    int chunk = (int)(SCAN_SMEM_BYTES / (2 * per_token));
    chunk = chunk < 1 ? 1 : (chunk > 16 ? 16 : chunk);
    const size_t smem = 2 * per_token * chunk;
    if (smem > 48 * 1024) BL_FAIL("bl_recurrent_scan: %d key channels need %zu bytes of shared memory a token", dk, per_token);
    // 16-byte copies where every row of q, k and z starts on a 16-byte boundary
    const int vec = dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ldz % 4 == 0 &&
                    (((uintptr_t)q | (uintptr_t)k | (uintptr_t)z) & 15) == 0;
    dim3 grid((dv + cols_blk - 1) / cols_blk, H, R * nc);
    const dim3 grid_wide((dv + dk + cols_blk - 1) / cols_blk, H, R * nc);     // the delta rule's first pass
    cudaStream_t s = (cudaStream_t)stream;
    if (rule != BL_RULE_GLA && rule != BL_RULE_DELTA && rule != BL_RULE_BONUS) BL_FAIL("bl_recurrent_scan: unknown rule %d", rule);
    if (rk4 > 0) {                                     // a lane's rows are whole groups of four
        const bool dl = rule == BL_RULE_DELTA;
        float* part_s = scratch;                                                 // [R, nc, H, dk, dv]
        float* part_p = scratch ? scratch + (size_t)R * nc * H * dk * dv : nullptr;   // [R, nc, H, dk] or, delta rule, [R, nc, H, dk, dk]
        float* part_start = (scratch && dl) ? part_p + (size_t)R * nc * H * dk * dk : nullptr;   // delta rule: [R, nc, H, dk, dv]
#define BL_SCAN(D, R4, PASS) BL_CUDA(bl_launch_dependent(recurrent_scan_vec_kernel<D, R4>, (D == BL_RULE_DELTA && PASS == 1) ? grid_wide : grid, dim3(WARPS * 32), smem, s, \
        q, ldq, k, ldk, v, ldv, z, ldz, beta, ldb, q_scale, state, (size_t)slot_stride, slots, cu_q, out, H, G, dk, dv, KS, chunk, vec, nc, PASS, \
        part_s, part_p, (const float*)part_start))
        for (int pass = (nc > 1 ? 1 : 2); pass <= 2; ++pass) {
            if (pass == 2 && nc > 1 && dl)
                BL_CUDA(bl_launch_dependent(scan_fold_matrix_kernel, dim3((dv + FOLD_COLS - 1) / FOLD_COLS, H, R), dim3(256), 0, s, state,
                                            (size_t)slot_stride, slots, cu_q, (const float*)part_s, (const float*)part_p, part_start,
                                            H, dk, dv, nc));
            switch (rk4) {
#define BL_SCAN_RULE(R4) do { if (dl) BL_SCAN(BL_RULE_DELTA, R4, pass); else if (rule == BL_RULE_BONUS) BL_SCAN(BL_RULE_BONUS, R4, pass); \
                                  else BL_SCAN(BL_RULE_GLA, R4, pass); } while (0)
                case 1: BL_SCAN_RULE(1); break;
                case 2: BL_SCAN_RULE(2); break;
                case 3: BL_SCAN_RULE(3); break;
                default: BL_SCAN_RULE(4); break;
#undef BL_SCAN_RULE
            }
        }
#undef BL_SCAN
        if (nc > 1 && !dl)
            BL_CUDA(bl_launch_dependent(scan_fold_kernel, dim3((dk * dv + 255) / 256, H, R), dim3(256), 0, s, state, (size_t)slot_stride, slots, cu_q,
                                        (const float*)part_s, (const float*)part_p, H, dk, dv, nc));
        BL_CHECK_LAUNCH("bl_recurrent_scan");
        return 0;
    }
    if (nc > 1) BL_FAIL("bl_recurrent_scan_parts: %d key channels cannot be cut into parts", dk);
    if (rule == BL_RULE_GLA)
        BL_CUDA(bl_launch_dependent(recurrent_scan_kernel<BL_RULE_GLA>, grid, dim3(WARPS * 32), smem, s, q, ldq, k, ldk, v, ldv, z, ldz, beta, ldb, q_scale,
            state, (size_t)slot_stride, slots, cu_q, out, H, G, dk, dv, KS, chunk, vec));
    else if (rule == BL_RULE_DELTA)
        BL_CUDA(bl_launch_dependent(recurrent_scan_kernel<BL_RULE_DELTA>, grid, dim3(WARPS * 32), smem, s, q, ldq, k, ldk, v, ldv, z, ldz, beta, ldb, q_scale,
            state, (size_t)slot_stride, slots, cu_q, out, H, G, dk, dv, KS, chunk, vec));
    else
        BL_CUDA(bl_launch_dependent(recurrent_scan_kernel<BL_RULE_BONUS>, grid, dim3(WARPS * 32), smem, s, q, ldq, k, ldk, v, ldv, z, ldz, beta, ldb, q_scale,
            state, (size_t)slot_stride, slots, cu_q, out, H, G, dk, dv, KS, chunk, vec));
    BL_CHECK_LAUNCH("bl_recurrent_scan");
    return 0;
}

extern "C" int bl_head_norm_gate(const float* o, const void* w, int w_dtype, const float* gate, int ld_gate, int gate_kind,
                                 void* y, int y_dtype, int T, int H, int dv, float eps, void* stream) {
    return bl_head_norm_gate_ext(o, dv, w, w_dtype, 0, nullptr, gate, ld_gate, gate_kind, y, y_dtype, T, H, dv, eps, stream);
}

extern "C" int bl_head_norm_gate_ext(const float* o, int o_head_stride, const void* w, int w_dtype, int w_per_head, const float* floor,
                                     const float* gate, int ld_gate, int gate_kind, void* y, int y_dtype, int T, int H, int dv, float eps,
                                     void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0 || (gate && ld_gate < H * dv) || o_head_stride < dv + (floor ? 1 : 0))
        BL_FAIL("bl_head_norm_gate: bad sizes H=%d dv=%d gate stride %d head stride %d", H, dv, ld_gate, o_head_stride);
    if (gate && gate_kind != BL_GATE_SIGMOID && gate_kind != BL_GATE_SILU) BL_FAIL("bl_head_norm_gate: unknown gate %d", gate_kind);
    const int items = T * H, blocks = (items + WARPS - 1) / WARPS;
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(head_norm_gate_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, s, o, o_head_stride, w, w_dtype, w_per_head,
                                    floor, gate, ld_gate, gate_kind, (float*)y, items, H, dv, eps));
    else if (y_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, s, o, o_head_stride, w, w_dtype,
                                    w_per_head, floor, gate, ld_gate, gate_kind, (__nv_bfloat16*)y, items, H, dv, eps));
    else
        BL_FAIL("bl_head_norm_gate: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_head_norm_gate");
    return 0;
}

extern "C" int bl_memory_gates(const float* proj, int ld, int off_k, int off_v, int off_i, int off_f, const void* bias_i, int bi_dtype,
                               const void* bias_f, int bf_dtype, float cap, float* state, long long slot_stride, long long off_m,
                               const int* slots, const int* cu_q, int R, int T, float* gates, float* decay, float* k_out, float* v_out,
                               int H, int dk, int dv, void* stream) {
    if (R <= 0 || T <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || !(cap > 0.f)) BL_FAIL("bl_memory_gates: bad sizes H=%d dk=%d dv=%d cap=%g", H, dk, dv, cap);
    if (R > 65535) BL_FAIL("bl_memory_gates: %d requests are too many for one launch", R);
    if (off_k + H * dk > ld || off_v + H * dv > ld || off_i + H > ld || off_f + H > ld) BL_FAIL("bl_memory_gates: columns do not fit rows of %d", ld);
    cudaStream_t s = (cudaStream_t)stream;
    BL_CUDA(bl_launch_dependent(memory_gate_chain_kernel, dim3(H, R), dim3(32), 0, s, proj, ld, off_i, off_f, bias_i, bi_dtype, bias_f, bf_dtype,
                                cap, state, (size_t)slot_stride, (size_t)off_m, slots, cu_q, gates, T, H));
    BL_CUDA(bl_launch_dependent(memory_expand_kernel, dim3(T), dim3(WARPS * 32), 0, s, proj, ld, off_k, off_v, (const float*)gates, decay, k_out,
                                v_out, T, H, dk, dv));
    BL_CHECK_LAUNCH("bl_memory_gates");
    return 0;
}

extern "C" int bl_shift_mix(const float* x, int ld, const float* mu, int n_mix, const float* prev, long long slot_stride,
                            const int* slots, const int* tok_req, const int* cu_q, void* out, int out_dtype, int T, int d, void* stream) {
    if (T <= 0) return 0;
    if (d <= 0 || ld < d || n_mix < 1) BL_FAIL("bl_shift_mix: bad sizes d=%d ld=%d mixes=%d", d, ld, n_mix);
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = d % 4 == 0 && ld % 4 == 0 && slot_stride % 4 == 0 &&
                    (((uintptr_t)x | (uintptr_t)mu | (uintptr_t)prev | (uintptr_t)out) & 15) == 0;
    if (out_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(shift_mix_kernel<float>, dim3(T), dim3(WARPS * 32), 0, s, x, ld, mu, n_mix, prev,
                                    (size_t)slot_stride, slots, tok_req, cu_q, (float*)out, T, d, vec));
    else if (out_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(shift_mix_kernel<__nv_bfloat16>, dim3(T), dim3(WARPS * 32), 0, s, x, ld, mu, n_mix, prev,
                                    (size_t)slot_stride, slots, tok_req, cu_q, (__nv_bfloat16*)out, T, d, vec));
    else
        BL_FAIL("bl_shift_mix: unknown output dtype %d", out_dtype);
    BL_CHECK_LAUNCH("bl_shift_mix");
    return 0;
}

extern "C" int bl_bonus_dot(const float* q, int ldq, const float* k, int ldk, const void* u, int u_dtype, float* out, int T, int H,
                            int dk, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dk <= 0 || ldq < H * dk || ldk < H * dk) BL_FAIL("bl_bonus_dot: bad sizes H=%d dk=%d", H, dk);
    const int items = T * H;
    BL_CUDA(bl_launch_dependent(bonus_dot_kernel, dim3((items + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, (cudaStream_t)stream, q, ldq, k, ldk,
                                u, u_dtype, out, items, H, dk));
    BL_CHECK_LAUNCH("bl_bonus_dot");
    return 0;
}

extern "C" int bl_conv_silu_unit(const float* x, int ld, const float* taps, int n_taps, const float* tail, long long slot_stride,
                                 const int* slots, const int* tok_req, const int* cu_q, float* y, int T, int C, int unit_heads,
                                 int scaled_heads, int dk, float q_scale, float unit_eps, void* stream) {
    return bl_conv_silu_unit_bias(x, ld, taps, n_taps, tail, slot_stride, slots, tok_req, cu_q, y, T, C, unit_heads, scaled_heads, dk,
                                  q_scale, unit_eps, nullptr, BL_F32, stream);
}

// The same with a bias per channel (null: none) that the convolution's sum starts from.
extern "C" int bl_conv_silu_unit_bias(const float* x, int ld, const float* taps, int n_taps, const float* tail, long long slot_stride,
                                      const int* slots, const int* tok_req, const int* cu_q, float* y, int T, int C, int unit_heads,
                                      int scaled_heads, int dk, float q_scale, float unit_eps, const void* bias, int bias_dtype,
                                      void* stream) {
    if (T <= 0) return 0;
    if (n_taps < 1 || n_taps > MAX_TAPS) BL_FAIL("bl_conv_silu_unit: %d taps, 1..%d are built", n_taps, MAX_TAPS);
    if (C <= 0 || ld < C || unit_heads * dk > C || scaled_heads > unit_heads)
        BL_FAIL("bl_conv_silu_unit: bad sizes C=%d ld=%d heads=%d of %d", C, ld, unit_heads, dk);
    BL_CUDA(bl_launch_dependent(conv_silu_unit_kernel, dim3(T), dim3(WARPS * 32), 0, (cudaStream_t)stream, x, ld, taps, n_taps, tail,
                                (size_t)slot_stride, slots, tok_req, cu_q, y, C, unit_heads, scaled_heads, dk, q_scale, unit_eps, bias, bias_dtype));
    BL_CHECK_LAUNCH("bl_conv_silu_unit");
    return 0;
}

extern "C" int bl_conv_tail_update(const float* x, int ld, int n_taps, float* tail, long long slot_stride, const int* slots,
                                   const int* cu_q, int R, int C, void* stream) {
    if (R <= 0 || n_taps <= 1) return 0;
    if (n_taps > MAX_TAPS) BL_FAIL("bl_conv_tail_update: %d taps, 1..%d are built", n_taps, MAX_TAPS);
    if (R > 65535) BL_FAIL("bl_conv_tail_update: %d requests are too many for one launch", R);
    dim3 grid((C + 127) / 128, R);
    BL_CUDA(bl_launch_dependent(conv_tail_update_kernel, grid, dim3(128), 0, (cudaStream_t)stream, x, ld, n_taps, tail,
                                (size_t)slot_stride, slots, cu_q, C));
    BL_CHECK_LAUNCH("bl_conv_tail_update");
    return 0;
}

extern "C" int bl_rope_decay_prep(const float* proj, int ld, int off_k, const int* positions, const float* inv_freq, int rot_half,
                                  const float* head_decay, float k_scale, float* q_out, float* k_out, float* decay_out, int T, int H,
                                  int dk, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dk <= 0 || rot_half < 0 || 2 * rot_half > dk || off_k < H * dk || ld < off_k + H * dk)
        BL_FAIL("bl_rope_decay_prep: bad sizes H=%d dk=%d rotated pairs=%d off_k=%d ld=%d", H, dk, rot_half, off_k, ld);
    BL_CUDA(bl_launch_dependent(rope_decay_prep_kernel, dim3(T), dim3(WARPS * 32), 0, (cudaStream_t)stream, proj, ld, off_k, positions,
                                inv_freq, rot_half, head_decay, k_scale, q_out, k_out, decay_out, H, dk));
    BL_CHECK_LAUNCH("bl_rope_decay_prep");
    return 0;
}

extern "C" int bl_ssd_prep(const float* raw, int ld_raw, const void* dt_bias, int bias_dtype, const float* rate, const float* x,
                           int ld_x, float* decay_out, float* v_out, int T, int H, int n_state, int dv, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || n_state <= 0 || dv <= 0 || ld_raw < H || ld_x < H * dv)
        BL_FAIL("bl_ssd_prep: bad sizes H=%d state=%d dv=%d ld_raw=%d ld_x=%d", H, n_state, dv, ld_raw, ld_x);
    BL_CUDA(bl_launch_dependent(ssd_prep_kernel, dim3(T), dim3(WARPS * 32), 0, (cudaStream_t)stream, raw, ld_raw, dt_bias, bias_dtype,
                                rate, x, ld_x, decay_out, v_out, H, n_state, dv));
    BL_CHECK_LAUNCH("bl_ssd_prep");
    return 0;
}

extern "C" int bl_gated_group_norm(const float* o, const float* x, int ld_x, const void* skip, int skip_dtype, int dv, const float* z,
                                   int ld_z, const void* w, int w_dtype, void* y, int y_dtype, int T, int width, int n_parts, float eps,
                                   void* stream) {
    if (T <= 0) return 0;
    if (width <= 0 || n_parts <= 0 || width % n_parts != 0 || (x && (dv <= 0 || width % dv != 0 || ld_x < width || !skip)) ||
        (z && ld_z < width))
        BL_FAIL("bl_gated_group_norm: bad sizes width=%d parts=%d dv=%d ld_x=%d ld_z=%d", width, n_parts, dv, ld_x, ld_z);
    if ((long long)T * n_parts > 2147483647LL) BL_FAIL("bl_gated_group_norm: %d rows in %d parts are more blocks than a launch takes", T, n_parts);
    const int blocks = T * n_parts;
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(gated_group_norm_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, s, o, x, ld_x, skip, skip_dtype, dv, z,
                                    ld_z, w, w_dtype, (float*)y, n_parts, width, eps));
    else if (y_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(gated_group_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, s, o, x, ld_x, skip, skip_dtype,
                                    dv, z, ld_z, w, w_dtype, (__nv_bfloat16*)y, n_parts, width, eps));
    else
        BL_FAIL("bl_gated_group_norm: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_gated_group_norm");
    return 0;
}
