// Shared helpers of the engine's CUDA sources: storage types, error reporting, warp reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

// Storage type codes of the C interface.
#define BL_F32 0
#define BL_BF16 1

// Epilogues of the matrix products.
#define BL_EPI_NONE 0      // out = acc
#define BL_EPI_BIAS 1      // out = acc + bias[n]
#define BL_EPI_RESIDUAL 2  // out (32-bit, in place) = out + acc
#define BL_EPI_SWIGLU 3    // out[m, n] = silu(acc_gate[m, n]) * acc_up[m, n]; W holds gate rows then up rows
#define BL_EPI_DECAY 4     // plain kernel only: out = exp(-coef[n / group] * softplus(sign * (acc + bias[n])))
#define BL_EPI_DECAY_EXP 5 // plain kernel only: out = exp(-exp(acc + bias[n])), optionally with tanh on x as it is read

// Which two dimensions of a head a rotary position encoding turns together (src/math.br:128-157, its `neox` argument).
#define BL_PAIRS_HALVES 0        // pair j = (j, j + n_rot / 2)
#define BL_PAIRS_INTERLEAVED 1   // pair j = (2j, 2j + 1)

void bl_set_error(const char* fmt, ...);

#define BL_FAIL(...) do { bl_set_error(__VA_ARGS__); return 1; } while (0)
#define BL_CHECK_LAUNCH(name) do { cudaError_t e_ = cudaGetLastError(); \
    if (e_ != cudaSuccess) BL_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e_)); } while (0)
#define BL_CUDA(call) do { cudaError_t e_ = (call); \
    if (e_ != cudaSuccess) BL_FAIL("%s failed: %s", #call, cudaGetErrorString(e_)); } while (0)

__device__ __forceinline__ float bl_load(const float* p) { return *p; }
__device__ __forceinline__ float bl_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void bl_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void bl_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Reads element i of an array whose storage type is known only at run time (small vectors:
// norm weights, biases; a tensor stored in 32-bit stays 32-bit beside bfloat16 matrices).
__device__ __forceinline__ float bl_load_any(const void* p, int dtype, size_t i) {
    return dtype == BL_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__device__ __forceinline__ float bl_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float bl_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x / (1 + exp(-x)), as src/math.br:232-233.
__device__ __forceinline__ float bl_silu(float x) { return x / (1.0f + expf(-x)); }
// The same with the hardware's exp2 and reciprocal units (relative error around 1e-6): for epilogues whose result
// is rounded to bfloat16 (2^-9) anyway and that evaluate it millions of times per step.
__device__ __forceinline__ float bl_silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Gated activations of a feed-forward, from the gate sum g and the up sum u of one hidden unit:
//   BL_GLU_SILU       g / (1 + e^-g) * u
//   BL_GLU_GELU_TANH  0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u
//   BL_GLU_CLAMPED    g' = min(g, limit), u' = clamp(u, -limit, limit):  g' / (1 + e^(-1.702 g')) * (u' + 1)
#define BL_GLU_SILU 0
#define BL_GLU_GELU_TANH 1
#define BL_GLU_CLAMPED 2
__device__ __forceinline__ float bl_glu(int kind, float g, float u, float limit) {
    if (kind == BL_GLU_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.79788456080286535588f * (g + 0.044715f * g * g * g))) * u;
    if (kind == BL_GLU_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return bl_silu(g) * u;
}
// The gated epilogue of a product (BL_EPI_SWIGLU) computes silu(gate) * up unless the product's `bias` argument, which
// that epilogue does not use otherwise, points to two 32-bit numbers {kind, limit}: then bl_glu(kind, gate, up, limit).
// bl_glu_fast: the same with the fast exponential and division of bl_silu_fast, for epilogues that round to bfloat16
// (0.5 g (1 + tanh(z)) = g / (1 + e^(-2z)), so each form is one exponential and one division).
__device__ __forceinline__ float bl_glu_fast(int kind, float g, float u, float limit) {
    if (kind == BL_GLU_GELU_TANH)
        return __fdividef(g, 1.0f + __expf(-1.59576912160573071176f * (g + 0.044715f * g * g * g))) * u;
    if (kind == BL_GLU_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fdividef(g, 1.0f + __expf(-1.702f * g)) * (u + 1.0f);
    }
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}
struct BlGluArgs { int kind; float limit; };
__device__ __forceinline__ BlGluArgs bl_glu_args(const void* two_numbers) {
    BlGluArgs a{BL_GLU_SILU, 0.f};
    if (two_numbers != nullptr) {
        const float* f = reinterpret_cast<const float*>(two_numbers);
        a.kind = (int)f[0];
        a.limit = f[1];
    }
    return a;
}

// xIELU with ap = softplus(p) and an = 1/2 + softplus(q) made ready: v > 0: ap v^2 + v / 2; v <= 0: an (e^v - 1 - v) + v / 2.
__device__ __forceinline__ float bl_xielu(float v, float ap, float an) {
    return v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
}

// What may follow the softmax of an attention row: a sink per head (a learned score whose exponential joins the
// denominator once, unscaled, with no value) and a gate per (token, head) whose sigmoid multiplies the row's output.
// bl_attn_tail returns the factor for the row's unnormalised output, given the row's maximum m in the base-2 domain
// (score * scale * log2 e) and the sum l of 2^(score - m). Null pointers: a plain 1 / l.
struct BlAttnTail { const void* sinks; int sink_dtype; const float* gate; int ld_gate; };
__device__ __forceinline__ float bl_attn_tail(const BlAttnTail& t, float m_log2, float l, size_t tok, int head) {
    float f = 1.f;
    if (t.sinks) {
        const float sk = bl_load_any(t.sinks, t.sink_dtype, head) * 1.4426950408889634f;
        const float mm = fmaxf(m_log2, sk);
        f = exp2f(m_log2 - mm);                        // a row without keys: 0
        l = l * f + exp2f(sk - mm);
    }
    float inv = l > 0.f ? f / l : 0.f;
    if (t.gate) inv *= 1.0f / (1.0f + expf(-t.gate[tok * (size_t)t.ld_gate + head]));
    return inv;
}

// Programmatic dependent launch. A kernel launched with bl_launch_dependent() may start while its predecessor
// on the stream is still running; whatever it does before bl_pdl_wait() must touch only data that no earlier
// kernel of the step writes (weights, the step's index arrays). bl_pdl_wait() returns once the predecessor has
// completed and its writes are visible. bl_pdl_trigger() lets the successor be scheduled as soon as every block
// of this kernel has issued it. Both are no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void bl_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void bl_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Asks for the 128-byte line at `p` to be brought into L2 (no register, no wait).
__device__ __forceinline__ void bl_prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" :: "l"(p)); }

// Brings rows [row0, row0 + n_rows) of a row-major matrix with `row_bytes` per row into L2, spread over the
// block's threads. Used before bl_pdl_wait() so that a kernel's weights stream from HBM while its
// predecessor is still running.
__device__ __forceinline__ void bl_prefetch_rows_l2(const void* base, size_t row0, int n_rows, size_t row_bytes,
                                                    size_t rows_total) {
    const int lines_per_row = (int)((row_bytes + 127) / 128);
    for (int i = threadIdx.x; i < n_rows * lines_per_row; i += blockDim.x) {
        const size_t r = row0 + i / lines_per_row;
        if (r < rows_total)
            bl_prefetch_l2(reinterpret_cast<const char*>(base) + r * row_bytes + (size_t)(i % lines_per_row) * 128);
    }
}

bool bl_pdl_enabled();

// The small kernels of a step all ask for the same split of an SM's memory between shared memory and L1.
// Kernels that want different splits cannot share an SM, so a chain of them would drain the SMs at every
// boundary and could never overlap under programmatic dependent launch. Set once per kernel.
template <typename... KArgs>
cudaError_t bl_same_carveout(void (*kernel)(KArgs...)) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

template <typename... KArgs, typename... Args>
cudaError_t bl_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args... args) {
    // one look-up per launch in a small table of kernels that already carry the carveout preference
    static thread_local const void* seen[64];
    static thread_local int n_seen = 0;
    bool known = false;
    for (int i = 0; i < n_seen; ++i) if (seen[i] == (const void*)kernel) { known = true; break; }
    if (!known) {
        cudaError_t e = bl_same_carveout(kernel);
        if (e != cudaSuccess) return e;
        if (n_seen < 64) seen[n_seen++] = (const void*)kernel;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose neighbouring blocks form clusters of `cluster_x` (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t bl_launch_dependent_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         unsigned cluster_x, Args... args) {
    static thread_local const void* seen[16];
    static thread_local int n_seen = 0;
    bool known = false;
    for (int i = 0; i < n_seen; ++i) if (seen[i] == (const void*)kernel) { known = true; break; }
    if (!known) {
        cudaError_t e = bl_same_carveout(kernel);
        if (e != cudaSuccess) return e;
        if (n_seen < 16) seen[n_seen++] = (const void*)kernel;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = cluster_x; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
