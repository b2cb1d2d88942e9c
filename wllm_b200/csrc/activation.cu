// Gated feed-forward activation on a fused [gate | up] row:
//     out[n, c] = act(gate[n, c]) * up[n, c],   gate = in[n, c], up = in[n, I + c]
// evaluated in 32-bit and rounded once.  act 0: tanh-approximated GELU
//     0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)));  act 1: SiLU  x / (1 + exp(-x));  act 2: ReLU  max(x, 0).
#include "common.cuh"

__device__ __forceinline__ float act_gelu_tanh(float x) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float act_silu(float x) { return x / (1.0f + expf(-x)); }
template <int ACT> __device__ __forceinline__ float act_apply(float x) {
    return ACT == 0 ? act_gelu_tanh(x) : ACT == 1 ? act_silu(x) : fmaxf(x, 0.f);
}
// the whole gated unit: act(g) * u for the plain activations, the clamped form for ACT 3
template <int ACT> __device__ __forceinline__ float gated_unit(float g, float u, float limit, float slope) {
    if (ACT == 3) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return (g / (1.0f + expf(-slope * g))) * (u + 1.0f);
    }
    return act_apply<ACT>(g) * u;
}

template <typename T, int ACT>
__global__ void gated_act_kernel(const T* __restrict__ in, T* __restrict__ out, int I, size_t total, float limit, float slope) {
    pdl_begin();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / I, c = idx % I;
        const float g = to_f32(in[n * 2 * I + c]), u = to_f32(in[n * 2 * I + I + c]);
        out[idx] = from_f32<T>(gated_unit<ACT>(g, u, limit, slope));
    }
}

// bfloat16 rows whose width is a multiple of 8: 16-byte loads and stores, grid (column blocks, rows)
template <int ACT>
__global__ void gated_act_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int I, float limit, float slope) {
    pdl_begin();
    const int n = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= I) return;
    const uint4 gv = *reinterpret_cast<const uint4*>(in + (size_t)n * 2 * I + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(in + (size_t)n * 2 * I + I + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        o2[i] = __floats2bfloat162_rn(gated_unit<ACT>(g.x, u.x, limit, slope), gated_unit<ACT>(g.y, u.y, limit, slope));
    }
    *reinterpret_cast<uint4*>(out + (size_t)n * I + c) = ov;
}

WLLM_API int wllm_gated_act_params(const void* in, void* out, int dtype, int act, int n, int I, float limit, float slope,
                                   cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (I <= 0) return WLLM_BAD_SIZE;
    if (act < 0 || act > 3) return WLLM_BAD_SIZE;
    if (dtype == WLLM_BF16 && I % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const dim3 grid((I / 8 + 127) / 128, n);
#define LAUNCH8(A) wllm_launch(gated_act_bf16x8_kernel<A>, grid, 128, 0, stream, (const bf16*)in, (bf16*)out, I, limit, slope)
        return act == 0 ? LAUNCH8(0) : act == 1 ? LAUNCH8(1) : act == 2 ? LAUNCH8(2) : LAUNCH8(3);
#undef LAUNCH8
    }
    const size_t total = (size_t)n * I;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
#define LAUNCH(T, A) wllm_launch(gated_act_kernel<T, A>, blocks, threads, 0, stream, (const T*)in, (T*)out, I, total, limit, slope)
    if (dtype == WLLM_BF16) return act == 0 ? LAUNCH(bf16, 0) : act == 1 ? LAUNCH(bf16, 1) : act == 2 ? LAUNCH(bf16, 2) : LAUNCH(bf16, 3);
    if (dtype == WLLM_F32) return act == 0 ? LAUNCH(float, 0) : act == 1 ? LAUNCH(float, 1) : act == 2 ? LAUNCH(float, 2) : LAUNCH(float, 3);
#undef LAUNCH
    return WLLM_BAD_DTYPE;
}

WLLM_API int wllm_gated_act(const void* in, void* out, int dtype, int act, int n, int I, cudaStream_t stream) {
    if (act == 3) return WLLM_BAD_SIZE;      // the clamped unit has constants: wllm_gated_act_params
    return wllm_gated_act_params(in, out, dtype, act, n, I, 0.f, 0.f, stream);
}

// x <- cap * tanh((x * scale) / cap); cap = 0: x <- x * scale
__global__ void tanh_cap_kernel(float* __restrict__ x, size_t total, float cap, float scale) {
    pdl_begin();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const float v = scale == 1.0f ? x[idx] : x[idx] * scale;
        x[idx] = cap > 0.f ? cap * tanhf(v / cap) : v;
    }
}

WLLM_API int wllm_scale_tanh_cap(float* x, long long total, float cap, float scale, cudaStream_t stream) {
    if (total <= 0) return WLLM_OK;
    if (!(cap >= 0.f)) return WLLM_BAD_SIZE;
    const long long want = (total + 255) / 256;
    return wllm_launch(tanh_cap_kernel, (int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream, x, (size_t)total, cap, scale);
}

WLLM_API int wllm_tanh_cap(float* x, long long total, float cap, cudaStream_t stream) {
    if (!(cap > 0.f)) return WLLM_BAD_SIZE;
    return wllm_scale_tanh_cap(x, total, cap, 1.0f, stream);
}

// A feed-forward unit without a gate: out = act(in), evaluated in 32-bit and rounded once.  act 0: relu(x)^2.
template <typename T>
__global__ void unit_act_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total) {
    pdl_begin();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(in[idx]), 0.f);
        out[idx] = from_f32<T>(v * v);
    }
}

WLLM_API int wllm_unit_act(const void* in, void* out, int dtype, int act, long long total, cudaStream_t stream) {
    if (total <= 0) return WLLM_OK;
    if (act != 0) return WLLM_BAD_SIZE;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == WLLM_BF16) return wllm_launch(unit_act_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, (size_t)total);
    if (dtype == WLLM_F32) return wllm_launch(unit_act_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, (size_t)total);
    return WLLM_BAD_DTYPE;
}

// The heads' outputs times a sigmoid gate: x[n, c] *= sigmoid(g[n, c]), c < width.  The gate's row comes as `parts` partial
// sums (slabs `part_stride` elements apart, added in order) or as one tensor; the sigmoid and the product are 32-bit, rounded once.
template <typename TX, typename TG>
__global__ void sigmoid_gate_kernel(TX* __restrict__ x, int x_stride, const TG* __restrict__ g, int g_stride, int parts,
                                    size_t part_stride, int n, int width) {
    pdl_begin();
    const size_t total = (size_t)n * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width, c = idx % width;
        const TG* src = g + t * g_stride + c;
        float z = to_f32(src[0]);
        for (int s = 1; s < parts; ++s) z += to_f32(src[(size_t)s * part_stride]);
        TX* dst = x + t * x_stride + c;
        *dst = from_f32<TX>(to_f32(*dst) * (1.0f / (1.0f + expf(-z))));
    }
}

WLLM_API int wllm_sigmoid_gate(void* x, int x_dtype, int x_stride, const void* g, int g_dtype, int g_stride, int parts,
                               long long part_stride, int n, int width, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (width <= 0 || parts < 1) return WLLM_BAD_SIZE;
    const long long want = ((long long)n * width + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
#define GO(TX, TG) wllm_launch(sigmoid_gate_kernel<TX, TG>, blocks, 256, 0, stream, (TX*)x, x_stride, (const TG*)g, g_stride, parts, \
                               (size_t)part_stride, n, width)
    if (x_dtype == WLLM_BF16 && g_dtype == WLLM_BF16) return GO(bf16, bf16);
    if (x_dtype == WLLM_BF16 && g_dtype == WLLM_F32) return GO(bf16, float);
    if (x_dtype == WLLM_F32 && g_dtype == WLLM_F32) return GO(float, float);
#undef GO
    return WLLM_BAD_DTYPE;
}

// A projection of the residual gates the token's own row of a table: out[t, c] = act(z[t, c]) * table[ids[t], c].  The
// projection's row comes as `parts` partial sums (added in order) or as one tensor; act 0: the tanh form of GELU.  32-bit, rounded once.
template <typename TZ, typename TT>
__global__ void token_gate_kernel(const TZ* __restrict__ z, int z_stride, int parts, size_t part_stride, const int* __restrict__ ids,
                                  const TT* __restrict__ table, int vocab, TT* __restrict__ out, int n, int dim) {
    pdl_begin();
    const size_t total = (size_t)n * dim;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / dim, c = idx % dim;
        const TZ* src = z + t * z_stride + c;
        float v = to_f32(src[0]);
        for (int s = 1; s < parts; ++s) v += to_f32(src[(size_t)s * part_stride]);
        const int id = min(max(ids[t], 0), vocab - 1);
        const float g = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        out[idx] = from_f32<TT>(g * to_f32(table[(size_t)id * dim + c]));
    }
}

WLLM_API int wllm_token_gate(const void* z, int z_dtype, int z_stride, int parts, long long part_stride, const int* ids,
                             const void* table, int t_dtype, int vocab, void* out, int act, int n, int dim, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (dim <= 0 || vocab <= 0 || parts < 1 || act != 0) return WLLM_BAD_SIZE;
    const long long want = ((long long)n * dim + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
#define GO(TZ, TT) wllm_launch(token_gate_kernel<TZ, TT>, blocks, 256, 0, stream, (const TZ*)z, z_stride, parts, (size_t)part_stride, ids, \
                               (const TT*)table, vocab, (TT*)out, n, dim)
    if (z_dtype == WLLM_BF16 && t_dtype == WLLM_BF16) return GO(bf16, bf16);
    if (z_dtype == WLLM_F32 && t_dtype == WLLM_BF16) return GO(float, bf16);
    if (z_dtype == WLLM_F32 && t_dtype == WLLM_F32) return GO(float, float);
#undef GO
    return WLLM_BAD_DTYPE;
}
