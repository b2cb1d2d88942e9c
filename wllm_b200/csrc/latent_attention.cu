// Attention over cached latent rows: what stands between the fused projection and the attention kernels.
//
// A token's cache row is [c | t | 0..]: c = rms(first `rank` columns of the down projection) * gain, the latent row from
// which every head's key and value are linear maps (k_h = Uk_h c, v_h = Uv_h c), and t, the `rot` columns behind them
// turned by the token's position, one key part shared by all heads.  A head's score is
//     q_h . [Uk_h c | t] = (Uk_h^T q_h[:dim]) . c + q_h[dim:] . t
// so with the queries mapped to a_h = [Uk_h^T q_h[:dim] | turned q_h[dim:]] attention runs over the cached rows themselves
// as one key/value head shared by all query heads, the values being the rows' first `rank` elements; a head's output
// o_h (rank elements) then passes Uv_h.  Nothing but the cached row is kept per token.
//
//   wllm_latent_prepare   one CTA a token: the cache row (norm in 32-bit from the projection's partial sums, the turn in
//                         32-bit), the queries' plain parts rounded for the product with Uk, their turned parts placed
//                         behind the columns that product will fill
//   wllm_head_linear_few  the same for bfloat16 steps of few tokens: a warp an output, the matrices read once.
//   wllm_head_linear      y[n, h, :N] = x[n, h, :K] W_h^T for every head h: the two maps above.  Every output is one
//                         ascending chain of fused multiply-adds over K in 32-bit, so a token's result does not depend on
//                         the step it is computed in.
#include "common.cuh"

__device__ __forceinline__ float value_at(const void* p, int dtype, size_t i) {
    return dtype == WLLM_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}

// fused row: [heads * (dim + rot) query columns | rank + rot down-projection columns] from column 0 of `fused`.
// With a latent row of the queries (q_rank > 0, no turning part): [q_rank columns | rank down-projection columns]; the first
// run is normed like the cache row, with a gain of its own, and goes to `cq_out` [n, q_rank] for the product that makes the
// queries; nothing of the queries is laid out here but the zeros behind every head's mapped part.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const TI* __restrict__ fused, int row_stride, int in_splits, size_t in_split_stride,
                      const int* __restrict__ positions, const int* __restrict__ slots, const float* __restrict__ inv_freq,
                      const void* __restrict__ gain, int gain_dtype, float eps, TO* __restrict__ pages, int page_size,
                      TO* __restrict__ q_plain, TO* __restrict__ q_mapped, int heads, int dim, int rot, int rot_dims,
                      int interleaved, int rank, int hd, int q_rank, const void* __restrict__ q_gain, TO* __restrict__ cq_out) {
    extern __shared__ float sm[];             // [rank] the latent columns, [half] sines, [half] cosines, [q_rank] the queries' latent columns
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dims >> 1;
    float* sn = sm + rank;
    float* cs = sn + half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
    pdl_wait();
    const TI* x = fused + (size_t)t * row_stride;
    auto in = [&](int c) {     // part 0 + part 1 + ... in order; sixteen loads are in flight at a time
        if (in_splits == 1) return to_f32(x[c]);
        float v = 0.f;
        for (int sp = 0; sp < in_splits; sp += 16) {
            float part[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) part[u] = sp + u < in_splits ? to_f32(x[(size_t)(sp + u) * in_split_stride + c]) : 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (sp + u < in_splits) v = (sp + u == 0) ? part[u] : v + part[u];
        }
        return v;
    };
    const int qw = q_rank > 0 ? q_rank : heads * (dim + rot);
    if (q_rank > 0) {
        float* qs = cs + half;
        float sq = 0.f;
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
            const float v = in(c);
            qs[c] = v;
            sq += v * v;
        }
        sq = block_sum(sq, scratch);
        const float inv_q = 1.0f / sqrtf(sq / (float)q_rank + eps);
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
            cq_out[(size_t)t * q_rank + c] = from_f32<TO>((qs[c] * inv_q) * value_at(q_gain, gain_dtype, c));
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = in(qw + c);
        sm[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);              // (its barriers also publish the sines and cosines)
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    // element e of a turned part whose plain values are given by `at`
    auto turned = [&](auto at, int e) {
        if (e >= rot_dims) return at(e);
        int j, partner;
        bool first;
        if (interleaved) { j = e >> 1; first = (e & 1) == 0; partner = first ? e + 1 : e - 1; }
        else { first = e < half; j = first ? e : e - half; partner = first ? e + half : e - half; }
        float y1, y2;
        if (first) { rotate_pair(at(e), at(partner), sn[j], cs[j], y1, y2); return y1; }
        rotate_pair(at(partner), at(e), sn[j], cs[j], y1, y2);
        return y2;
    };
    if (slot >= 0) {
        TO* dst = pages + ((size_t)(slot / page_size) * page_size + slot % page_size) * hd;
        for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f32<TO>((sm[c] * inv) * value_at(gain, gain_dtype, c));
        for (int e = threadIdx.x; e < hd - rank; e += blockDim.x)
            dst[rank + e] = e < rot ? from_f32<TO>(turned([&](int i) { return in(qw + rank + i); }, e)) : from_f32<TO>(0.f);
    }
    if (q_plain != nullptr && q_rank == 0)    // null: the next product reads the plain parts from the fused row itself
        for (int item = threadIdx.x; item < heads * dim; item += blockDim.x) {
            const int h = item / dim, c = item % dim;
            q_plain[(size_t)t * heads * dim + item] = from_f32<TO>(in(h * (dim + rot) + c));
        }
    const int tail = hd - rank;
    for (int item = threadIdx.x; item < heads * tail; item += blockDim.x) {
        const int h = item / tail, e = item % tail;
        const int base = h * (dim + rot) + dim;
        q_mapped[((size_t)t * heads + h) * hd + rank + e] =
            e < rot ? from_f32<TO>(turned([&](int i) { return in(base + i); }, e)) : from_f32<TO>(0.f);
    }
}

// fused [n, >= heads * (dim + rot) + rank + rot] (or `in_splits` 32-bit slabs), pages [page][1][slot][hd] with hd >= rank + rot,
// q_plain [n, heads * dim] (or null), q_mapped [n, heads * hd] (columns rank .. hd of every head are written here), gain [rank].
WLLM_API int wllm_latent_prepare(const void* fused, int in_dtype, int row_stride, int in_splits, long long in_split_stride,
                                 const int* positions, const int* slots, const float* inv_freq, const void* gain, int gain_dtype,
                                 float eps, void* pages, int page_size, void* q_plain, void* q_mapped, int out_dtype, int n,
                                 int heads, int dim, int rot, int rot_dims, int interleaved, int rank, int hd, int q_rank,
                                 const void* q_gain, void* cq_out, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (heads <= 0 || dim <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || rank <= 0 || hd < rank + rot ||
        page_size <= 0 || in_splits < 1)
        return WLLM_BAD_SIZE;
    if (q_rank < 0 || (q_rank > 0 && (rot != 0 || q_gain == nullptr || cq_out == nullptr))) return WLLM_BAD_SIZE;
    if (gain_dtype != WLLM_BF16 && gain_dtype != WLLM_F32) return WLLM_BAD_DTYPE;
    const size_t smem = ((size_t)rank + rot_dims + q_rank) * sizeof(float);
    if (smem > 48 * 1024) return WLLM_BAD_SIZE;
#define GO(TI, TO) wllm_launch(latent_prepare_kernel<TI, TO>, n, 256, smem, stream, (const TI*)fused, row_stride, in_splits, \
        (size_t)in_split_stride, positions, slots, inv_freq, gain, gain_dtype, eps, (TO*)pages, page_size, (TO*)q_plain, \
        (TO*)q_mapped, heads, dim, rot, rot_dims, interleaved, rank, hd, q_rank, q_gain, (TO*)cq_out)
    if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16) return GO(bf16, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_BF16) return GO(float, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_F32) return GO(float, float);
#undef GO
    return WLLM_BAD_DTYPE;
}

// ---------------------------------------------------------------------------------------------------
// y[t, h, j] = sum_k x[t, h, k] * w[h, j, k]: tiles of 64 tokens by 64 outputs of one head, 16 columns of K a step
// through shared memory, 4 x 4 outputs a thread, every output one chain over k in ascending order.
// ---------------------------------------------------------------------------------------------------
constexpr int HL_T = 64, HL_K = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, int x_row, int x_head, const T* __restrict__ w, T* __restrict__ y, int y_row,
                   int y_head, int n, int N, int K) {
    __shared__ float xs[HL_K][HL_T + 4], ws[HL_K][HL_T + 4];
    pdl_begin();
    const int h = blockIdx.z, t0 = blockIdx.y * HL_T, j0 = blockIdx.x * HL_T;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // outputs j0 + tx * 4 .., tokens t0 + ty * 4 ..
    const T* xh = x + (size_t)h * x_head;
    const T* wh = w + (size_t)h * N * K;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HL_K) {
        for (int idx = threadIdx.x; idx < HL_T * HL_K; idx += blockDim.x) {
            const int r = idx / HL_K, k = idx % HL_K;
            const bool in_k = k0 + k < K;
            xs[k][r] = (in_k && t0 + r < n) ? to_f32(xh[(size_t)(t0 + r) * x_row + k0 + k]) : 0.f;
            ws[k][r] = (in_k && j0 + r < N) ? to_f32(wh[(size_t)(j0 + r) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
        const int kn = min(HL_K, K - k0);     // columns past K would add fma(0, 0, acc) = acc; they are left out all the same
        for (int k = 0; k < kn; ++k) {
            float xv[4], wv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) { xv[a] = xs[k][ty * 4 + a]; wv[a] = ws[k][tx * 4 + a]; }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(xv[a], wv[b], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int t = t0 + ty * 4 + a;
        if (t >= n) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int j = j0 + tx * 4 + b;
            if (j < N) y[(size_t)t * y_row + (size_t)h * y_head + j] = from_f32<T>(acc[a][b]);
        }
    }
}

// The same map for bfloat16 steps of few tokens (decoded tokens), where the matrices are what is read: a warp an output
// (head h, column j) for up to HF_T tokens at once.  The lanes stride over K with 16-byte loads of w, each token's sum is
// reduced over the lanes in a fixed order, so a token's result does not depend on the other tokens of the step.
constexpr int HF_T = 8;

__global__ void __launch_bounds__(256)
head_linear_few_kernel(const bf16* __restrict__ x, int x_row, int x_head, const bf16* __restrict__ w, bf16* __restrict__ y,
                       int y_row, int y_head, int n, int heads, int N, int K) {
    pdl_begin();
    const int lane = threadIdx.x & 31;
    const long long out = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (out >= (long long)heads * N) return;
    const int h = (int)(out / N), j = (int)(out % N);
    const int t0 = blockIdx.y * HF_T, nt = min(HF_T, n - t0);
    const bf16* wr = w + ((size_t)h * N + j) * K;
    const bf16* xh = x + (size_t)t0 * x_row + (size_t)h * x_head;
    float acc[HF_T];
#pragma unroll
    for (int t = 0; t < HF_T; ++t) acc[t] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wr + k);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int t = 0; t < HF_T; ++t) {
            if (t >= nt) continue;
            const uint4 xv = *reinterpret_cast<const uint4*>(xh + (size_t)t * x_row + k);
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(x2[e]), b = __bfloat1622float2(w2[e]);
                acc[t] = fmaf(a.x, b.x, acc[t]);
                acc[t] = fmaf(a.y, b.y, acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < HF_T; ++t) {
        float v = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && t < nt) y[(size_t)(t0 + t) * y_row + (size_t)h * y_head + j] = __float2bfloat16_rn(v);
    }
}

// bfloat16, K and the strides of x in steps of 8 elements, 16-byte aligned x and w: steps of up to `few` tokens run a warp an output.
WLLM_API int wllm_head_linear_few(const void* x, int x_row, int x_head, const void* w, void* y, int y_row, int y_head, int n,
                                  int heads, int N, int K, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (heads <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || x_row % 8 != 0 || x_head % 8 != 0) return WLLM_BAD_SIZE;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return WLLM_BAD_ALIGN;
    const long long ctas = ((long long)heads * N + 7) / 8;
    const int token_blocks = (n + HF_T - 1) / HF_T;
    if (ctas > 0x7fffffffLL || token_blocks > 65535) return WLLM_BAD_SIZE;
    return wllm_launch(head_linear_few_kernel, dim3((unsigned)ctas, token_blocks), 256, 0, stream, (const bf16*)x, x_row, x_head,
                       (const bf16*)w, (bf16*)y, y_row, y_head, n, heads, N, K);
}

// x: element (t, h, k) at t * x_row + h * x_head + k; w [heads, N, K] contiguous; y: element (t, h, j) at t * y_row + h * y_head + j.
WLLM_API int wllm_head_linear(const void* x, int x_row, int x_head, const void* w, void* y, int y_row, int y_head, int dtype,
                              int n, int heads, int N, int K, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (heads <= 0 || heads > 65535 || N <= 0 || K <= 0) return WLLM_BAD_SIZE;
    const dim3 grid((N + HL_T - 1) / HL_T, (n + HL_T - 1) / HL_T, heads);
    if (grid.y > 65535) return WLLM_BAD_SIZE;
    if (dtype == WLLM_BF16)
        return wllm_launch(head_linear_kernel<bf16>, grid, 256, 0, stream, (const bf16*)x, x_row, x_head, (const bf16*)w, (bf16*)y,
                           y_row, y_head, n, N, K);
    if (dtype == WLLM_F32)
        return wllm_launch(head_linear_kernel<float>, grid, 256, 0, stream, (const float*)x, x_row, x_head, (const float*)w,
                           (float*)y, y_row, y_head, n, N, K);
    return WLLM_BAD_DTYPE;
}
