// Root-mean-square norm over the 32-bit residual stream, with the pending branch
// output folded in first:
//     r = resid[row] (+ delta[row]);  resid[row] = r  (when a delta is given);
//     out[i] = r * (1 / sqrt(mean(r^2) + eps)) * (offset + w)
// `delta` may come as `delta_splits` partial sums (slabs `delta_split_stride` elements apart, as the
// split-K matrix product leaves them); they are added in slab order.
// All arithmetic is 32-bit; `out` is rounded once to the matrix type.  With `rows`
// the kernel reads row rows[i] and writes row i (the final norm at the places whose
// logits are wanted) and leaves the residual untouched.  One block per row; the sum
// of squares is reduced in a fixed order that depends on nothing but the row.
// With `center` the row's mean is taken off first (a layer norm without a bias):
//     out[i] = (r - mean(r)) / sqrt(mean((r - mean)^2) + eps) * (offset + w)
// Without a gain (`w` null) nothing is normed: out = r rounded to the matrix type, which is how a sublayer that reads
// the residual as it is gets its input (the pending add is still folded in).
// `wllm_branch_norm` norms a branch output (or two of them) that is not yet part of the residual:
//     out = factor * (norm(a) * wa  [+ norm(b) * wb]),   32-bit out
// which is the norm behind a sublayer of a block that norms on both sides, and the mean of two mixers.
#include "common.cuh"

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}

// v += part 0 + part 1 + ... in that order.  The loads of sixteen parts are issued together (they do not
// depend on one another); only the additions are in sequence.
template <typename TD, int VEC>
__device__ __forceinline__ void add_parts(float (&v)[4], const TD* __restrict__ d, int parts, size_t stride) {
    if (parts == 1) {      // the common case: one tensor to add
        float dv[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC == 4) load4(d, dv); else dv[0] = to_f32(d[0]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] += dv[k];
        return;
    }
    for (int sp = 0; sp < parts; sp += 16) {
        float dv[16][4];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            dv[u][0] = dv[u][1] = dv[u][2] = dv[u][3] = 0.f;
            if (sp + u < parts) {
                if (VEC == 4) load4(d + (size_t)(sp + u) * stride, dv[u]);
                else dv[u][0] = to_f32(d[(size_t)(sp + u) * stride]);
            }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u)
            if (sp + u < parts) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) v[k] += dv[u][k];
            }
    }
}

// VEC = 4: rows whose width is a multiple of 4 are read and written four elements at a time.
// VPT = 1, 2 or 4: the whole row fits in registers with that many vectors a thread, and memory is passed
// over once; VPT = 0: wider rows (or VEC = 1) take two passes.
template <typename TD, typename TW, typename TO, int VEC, int VPT>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, int delta_splits,
                               size_t delta_split_stride, const TW* __restrict__ w, float eps, float offset,
                               TO* __restrict__ out, const int* __restrict__ rows, int H, int center) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    constexpr bool one_pass = VEC == 4 && VPT > 0;
    constexpr int NV = VPT > 0 ? VPT : 1;
    const bool plain = w == nullptr;      // no gain: the row goes out as it is
    float wv[NV][4];
    if (one_pass) {          // the gain is written by no kernel: it is read while the predecessor still runs
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            wv[k][0] = wv[k][1] = wv[k][2] = wv[k][3] = 0.f;
            if (c < H && !plain) load4(w + c, wv[k]);
        }
    }
    pdl_wait();
    const int i = blockIdx.x;
    const int row = rows ? rows[i] : i;
    float* r = resid + (size_t)row * H;
    const TD* d = delta ? delta + (size_t)row * H : nullptr;
    const bool write_back = (d != nullptr) && (rows == nullptr);
    TO* o = out + (size_t)i * H;
    if (one_pass) {
        float v[NV][4];
        float ss = 0.f, sum = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.f;
            if (c < H) {
                load4(r + c, v[k]);
                if (d) add_parts<TD, 4>(v[k], d + c, delta_splits, delta_split_stride);
#pragma unroll
                for (int e = 0; e < 4; ++e) sum += v[k][e];
            }
        }
        if (plain) {
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int c = (threadIdx.x + k * blockDim.x) * 4;
                if (c < H) {
                    if (write_back) store4(r + c, v[k]);
                    store4(o + c, v[k]);
                }
            }
            return;
        }
        const float mean = center ? block_sum(sum, scratch) / (float)H : 0.f;     // (x - 0) is x, bit for bit
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            if (c < H) {
#pragma unroll
                for (int e = 0; e < 4; ++e) ss += (v[k][e] - mean) * (v[k][e] - mean);
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            if (c < H) {
                float y[4];
                if (write_back) store4(r + c, v[k]);
#pragma unroll
                for (int e = 0; e < 4; ++e) y[e] = ((v[k][e] - mean) * inv) * (offset + wv[k][e]);
                store4(o + c, y);
            }
        }
        return;
    }
    if (plain) {
        for (int c = threadIdx.x * VEC; c < H; c += blockDim.x * VEC) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (VEC == 4) load4(r + c, v); else v[0] = r[c];
            if (d) add_parts<TD, VEC>(v, d + c, delta_splits, delta_split_stride);
            if (write_back) {
                if (VEC == 4) store4(r + c, v); else r[c] = v[0];
            }
            if (VEC == 4) store4(o + c, v); else o[c] = from_f32<TO>(v[0]);
        }
        return;
    }
    float mean = 0.f;
    if (center) {
        float sum = 0.f;
        for (int c = threadIdx.x * VEC; c < H; c += blockDim.x * VEC) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (VEC == 4) load4(r + c, v); else v[0] = r[c];
            if (d) add_parts<TD, VEC>(v, d + c, delta_splits, delta_split_stride);
#pragma unroll
            for (int k = 0; k < VEC; ++k) sum += v[k];
        }
        mean = block_sum(sum, scratch) / (float)H;
    }
    float ss = 0.f;
    for (int c = threadIdx.x * VEC; c < H; c += blockDim.x * VEC) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC == 4) load4(r + c, v); else v[0] = r[c];
        if (d) add_parts<TD, VEC>(v, d + c, delta_splits, delta_split_stride);
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss += (v[k] - mean) * (v[k] - mean);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x * VEC; c < H; c += blockDim.x * VEC) {
        float v[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC == 4) { load4(r + c, v); load4(w + c, wv); }
        else { v[0] = r[c]; wv[0] = to_f32(w[c]); }
        if (d) add_parts<TD, VEC>(v, d + c, delta_splits, delta_split_stride);
        if (write_back) {
            if (VEC == 4) store4(r + c, v); else r[c] = v[0];
        }
        float y[4];
#pragma unroll
        for (int k = 0; k < VEC; ++k) y[k] = ((v[k] - mean) * inv) * (offset + wv[k]);
        if (VEC == 4) store4(o + c, y); else o[c] = from_f32<TO>(y[0]);
    }
}

template <typename TD, typename TW>
static int launch_out(float* resid, const void* delta, int delta_splits, size_t delta_split_stride, const void* w, float eps,
                      float offset, void* out, int out_dtype, const int* rows, int n, int H, int center, cudaStream_t stream) {
    const bool vec = H % 4 == 0 && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)delta & 15) == 0 &&
                     ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0 && delta_split_stride % 4 == 0;
    const int per = vec ? 4 : 1;
    const int threads = H / per >= 512 ? 512 : (H / per >= 256 ? 256 : 128);   // one vector a thread up to 2048 columns
    const int vpt = !vec ? 0 : (H <= threads * 4 ? 1 : (H <= threads * 8 ? 2 : (H <= threads * 16 ? 4 : 0)));
#define GO(TO, V, P) wllm_launch(rmsnorm_kernel<TD, TW, TO, V, P>, n, threads, 0, stream, resid, (const TD*)delta, delta_splits, \
                       delta_split_stride, (const TW*)w, eps, offset, (TO*)out, rows, H, center)
#define PICK(TO) (vpt == 1 ? GO(TO, 4, 1) : vpt == 2 ? GO(TO, 4, 2) : vpt == 4 ? GO(TO, 4, 4) : vec ? GO(TO, 4, 0) : GO(TO, 1, 0))
    if (out_dtype == WLLM_BF16) return PICK(bf16);
    if (out_dtype == WLLM_F32) return PICK(float);
#undef PICK
#undef GO
#undef GO2
    return WLLM_BAD_DTYPE;
}

// center 0: root-mean-square norm; 1: the mean is taken off first (layer norm without a bias).
WLLM_API int wllm_norm(float* resid, const void* delta, int delta_dtype, int delta_splits, long long delta_split_stride,
                       const void* w, int w_dtype, float eps, float offset, int center, void* out, int out_dtype,
                       const int* rows, int n, int H, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || delta_splits < 1 || delta_split_stride < 0) return WLLM_BAD_SIZE;
    const bool dbf = delta_dtype == WLLM_BF16, wbf = w_dtype == WLLM_BF16;
    if ((delta_dtype != WLLM_BF16 && delta_dtype != WLLM_F32) || (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32)) return WLLM_BAD_DTYPE;
    center = center ? 1 : 0;
    if (dbf && wbf) return launch_out<bf16, bf16>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, center, stream);
    if (dbf && !wbf) return launch_out<bf16, float>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, center, stream);
    if (!dbf && wbf) return launch_out<float, bf16>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, center, stream);
    return launch_out<float, float>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, center, stream);
}

WLLM_API int wllm_rmsnorm(float* resid, const void* delta, int delta_dtype, int delta_splits, long long delta_split_stride,
                          const void* w, int w_dtype, float eps, float offset, void* out, int out_dtype, const int* rows,
                          int n, int H, cudaStream_t stream) {
    return wllm_norm(resid, delta, delta_dtype, delta_splits, delta_split_stride, w, w_dtype, eps, offset, 0, out, out_dtype,
                     rows, n, H, stream);
}

// ---------------------------------------------------------------------------------------------------
// The norm of a branch output (or of two, added): one block per row, every pass reads the parts again
// (they lie in the L2) and adds them in slab order, so that no row length is too long for it.
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float any_at(const void* p, int dtype, size_t i) {
    return dtype == WLLM_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}
// part 0 + part 1 + ... in that order (several parts are always 32-bit slabs); sixteen loads are in flight at a time,
// only the additions are a chain
// MULTI false: the kernel was launched for single tensors and carries none of the code for parts (the registers of
// sixteen loads in flight cost the many-row launches their occupancy: a prompt's branch norm took 49 us with them, 37 without)
template <bool MULTI>
__device__ __forceinline__ float parts_at(const void* p, int dtype, int parts, size_t stride, size_t i) {
    if (!MULTI || parts == 1) return any_at(p, dtype, i);
    const float* f = reinterpret_cast<const float*>(p) + i;
    float v = 0.f;
    for (int s0 = 0; s0 < parts; s0 += 16) {
        float part[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) part[u] = s0 + u < parts ? f[(size_t)(s0 + u) * stride] : 0.f;
#pragma unroll
        for (int u = 0; u < 16; ++u)
            if (s0 + u < parts) v = (s0 + u == 0) ? part[u] : v + part[u];
    }
    return v;
}
// (mean, 1 / sqrt(var + eps)) of one row of a branch
template <bool MULTI>
__device__ __forceinline__ void branch_stats(const void* p, int dtype, int parts, size_t stride, size_t row0, int H, int center,
                                             float eps, float* scratch, float& mean, float& inv) {
    mean = 0.f;
    if (center) {
        float sum = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) sum += parts_at<MULTI>(p, dtype, parts, stride, row0 + c);
        mean = block_sum(sum, scratch) / (float)H;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = parts_at<MULTI>(p, dtype, parts, stride, row0 + c) - mean;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / (float)H + eps);
}

template <bool MULTI>
__global__ void branch_norm_kernel(const void* __restrict__ a, int a_dtype, int a_parts, size_t a_stride, const void* __restrict__ wa,
                                   const void* __restrict__ b, int b_dtype, int b_parts, size_t b_stride, const void* __restrict__ wb,
                                   int w_dtype, float eps, int center, float factor, float* __restrict__ out, int H, float offset) {
    __shared__ float scratch[32];
    pdl_begin();
    const size_t row0 = (size_t)blockIdx.x * H;
    float mean_a, inv_a, mean_b = 0.f, inv_b = 0.f;
    branch_stats<MULTI>(a, a_dtype, a_parts, a_stride, row0, H, center, eps, scratch, mean_a, inv_a);
    if (b) branch_stats<MULTI>(b, b_dtype, b_parts, b_stride, row0, H, center, eps, scratch, mean_b, inv_b);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float y = ((parts_at<MULTI>(a, a_dtype, a_parts, a_stride, row0 + c) - mean_a) * inv_a) * (offset + any_at(wa, w_dtype, c));
        if (b) y += ((parts_at<MULTI>(b, b_dtype, b_parts, b_stride, row0 + c) - mean_b) * inv_b) * (offset + any_at(wb, w_dtype, c));
        out[row0 + c] = y * factor;
    }
}

// out[n, H] (32-bit) = factor * (norm(a) * wa + norm(b) * wb); b and wb may be null.  a and b are [n, H] tensors of either
// element type or `parts` 32-bit slabs `stride` elements apart; the gains share one element type and are offset + w.
WLLM_API int wllm_branch_norm_offset(const void* a, int a_dtype, int a_parts, long long a_stride, const void* wa,
                                     const void* b, int b_dtype, int b_parts, long long b_stride, const void* wb, int w_dtype,
                                     float eps, int center, float factor, float offset, float* out, int n, int H,
                                     cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || a_parts < 1 || (b && b_parts < 1)) return WLLM_BAD_SIZE;
    if ((a_dtype != WLLM_BF16 && a_dtype != WLLM_F32) || (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32) ||
        (b && b_dtype != WLLM_BF16 && b_dtype != WLLM_F32))
        return WLLM_BAD_DTYPE;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (a_parts > 1 || (b && b_parts > 1))
        return wllm_launch(branch_norm_kernel<true>, n, threads, 0, stream, a, a_dtype, a_parts, (size_t)a_stride, wa, b, b_dtype,
                           b_parts, (size_t)b_stride, wb, w_dtype, eps, center ? 1 : 0, factor, out, H, offset);
    return wllm_launch(branch_norm_kernel<false>, n, threads, 0, stream, a, a_dtype, a_parts, (size_t)a_stride, wa, b, b_dtype,
                       b_parts, (size_t)b_stride, wb, w_dtype, eps, center ? 1 : 0, factor, out, H, offset);
}

WLLM_API int wllm_branch_norm(const void* a, int a_dtype, int a_parts, long long a_stride, const void* wa,
                              const void* b, int b_dtype, int b_parts, long long b_stride, const void* wb, int w_dtype,
                              float eps, int center, float factor, float* out, int n, int H, cudaStream_t stream) {
    return wllm_branch_norm_offset(a, a_dtype, a_parts, a_stride, wa, b, b_dtype, b_parts, b_stride, wb, w_dtype, eps, center,
                                   factor, 0.f, out, n, H, stream);
}

// ---------------------------------------------------------------------------------------------------
// A block that norms behind its sublayers as well as in front, in one kernel a row:
//     u   = a                                             (one branch), or
//           factor * (rms(a) * wa + rms(b) * wb)          (two mixers side by side, each normed over the width)
//     r  += norm_p(u) * (offset_p + wp)                   (the norm behind the sublayer; center_p: layer norm)
//     out = norm(r) * (offset + w)                        (the norm in front of the next sublayer, or the model's last;
//                                                          w null: out = r, for a sublayer that reads the residual as it is)
// The row lives in shared memory between the passes (H floats); every sum is a block sum in a fixed order.
// With `rows` the residual is read at rows[i] and left as it is (the last norm at the places whose logits are wanted).
// ---------------------------------------------------------------------------------------------------
template <typename TO, bool MULTI>
__global__ void sandwich_norm_kernel(float* __restrict__ resid, const void* __restrict__ a, int a_dtype, int a_parts, size_t a_stride,
                                     const void* __restrict__ wa, const void* __restrict__ b, int b_dtype, int b_parts,
                                     size_t b_stride, const void* __restrict__ wb, float inner_eps, float factor,
                                     const void* __restrict__ wp, int center_p, float eps_p, const void* __restrict__ w,
                                     float offset, int center, float eps, int w_dtype, TO* __restrict__ out,
                                     const int* __restrict__ rows, int H, float offset_p) {
    extern __shared__ float row_s[];          // [H] the row between the passes; with two branches [H] more for the second
    __shared__ float scratch[32];
    pdl_begin();
    const int i = blockIdx.x;
    const size_t row0 = (size_t)(rows ? rows[i] : i) * H;
    float* row_b = row_s + H;
    float inv_a = 1.f, inv_b = 1.f;
    // the branches' parts are added once and kept: every later pass reads shared memory
    float ssa = 0.f, ssb = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = parts_at<MULTI>(a, a_dtype, a_parts, a_stride, row0 + c);
        row_s[c] = x;
        ssa += x * x;
        if (b) { const float y = parts_at<MULTI>(b, b_dtype, b_parts, b_stride, row0 + c); row_b[c] = y; ssb += y * y; }
    }
    if (wa) {
        inv_a = 1.0f / sqrtf(block_sum(ssa, scratch) / (float)H + inner_eps);
        if (b) inv_b = 1.0f / sqrtf(block_sum(ssb, scratch) / (float)H + inner_eps);
    }
    float sum = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float u = row_s[c];
        if (wa) {
            u = (u * inv_a) * any_at(wa, w_dtype, c);
            if (b) u += (row_b[c] * inv_b) * any_at(wb, w_dtype, c);
            u *= factor;
        }
        row_s[c] = u;
        sum += u;
    }
    float mean = center_p ? block_sum(sum, scratch) / (float)H : 0.f;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) ss += (row_s[c] - mean) * (row_s[c] - mean);
    float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps_p);
    sum = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = resid[row0 + c] + ((row_s[c] - mean) * inv) * (offset_p + any_at(wp, w_dtype, c));
        if (!rows) resid[row0 + c] = x;
        row_s[c] = x;
        sum += x;
    }
    TO* o = out + (size_t)i * H;
    if (w == nullptr) {           // every thread reads back what it wrote itself
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f32<TO>(row_s[c]);
        return;
    }
    mean = center ? block_sum(sum, scratch) / (float)H : 0.f;
    ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) ss += (row_s[c] - mean) * (row_s[c] - mean);
    inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        o[c] = from_f32<TO>(((row_s[c] - mean) * inv) * (offset + any_at(w, w_dtype, c)));
}

// a, b: branch outputs [n, H] of either element type, or `parts` 32-bit slabs `stride` elements apart; wa null: a is taken as
// it is (b, wb unused); all gains (wa, wb, wp, w) share one element type.
// offset_p: the gain of the norm behind the sublayer is offset_p + wp; w null: the second norm is left out (out = r).
WLLM_API int wllm_sandwich_norm_offset(float* resid, const void* a, int a_dtype, int a_parts, long long a_stride, const void* wa,
                                       const void* b, int b_dtype, int b_parts, long long b_stride, const void* wb, float inner_eps,
                                       float factor, const void* wp, float offset_p, int center_p, float eps_p, const void* w,
                                       float offset, int center, float eps, int w_dtype, void* out, int out_dtype,
                                       const int* rows, int n, int H, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || H > 24 * 1024 || a_parts < 1 || (b && b_parts < 1) || (b && !wa)) return WLLM_BAD_SIZE;
    if ((a_dtype != WLLM_BF16 && a_dtype != WLLM_F32) || (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32) ||
        (b && b_dtype != WLLM_BF16 && b_dtype != WLLM_F32))
        return WLLM_BAD_DTYPE;
    const size_t smem = (size_t)(b ? 2 : 1) * H * sizeof(float);
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaSuccess;
#define RAISE(K) if (e == cudaSuccess) e = cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024)
        RAISE((sandwich_norm_kernel<bf16, true>)); RAISE((sandwich_norm_kernel<bf16, false>));
        RAISE((sandwich_norm_kernel<float, true>)); RAISE((sandwich_norm_kernel<float, false>));
#undef RAISE
        if (e != cudaSuccess) return 1000 + (int)e;
        raised = true;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool multi = a_parts > 1 || (b && b_parts > 1);
#define GO2(TO, M) wllm_launch(sandwich_norm_kernel<TO, M>, n, threads, smem, stream, resid, a, a_dtype, a_parts, (size_t)a_stride, wa, b, \
        b_dtype, b_parts, (size_t)b_stride, wb, inner_eps, factor, wp, center_p ? 1 : 0, eps_p, w, offset, center ? 1 : 0, eps, \
        w_dtype, (TO*)out, rows, H, offset_p)
#define GO(TO) (multi ? GO2(TO, true) : GO2(TO, false))
    if (out_dtype == WLLM_BF16) return GO(bf16);
    if (out_dtype == WLLM_F32) return GO(float);
#undef GO
#undef GO2
    return WLLM_BAD_DTYPE;
}

WLLM_API int wllm_sandwich_norm(float* resid, const void* a, int a_dtype, int a_parts, long long a_stride, const void* wa,
                                const void* b, int b_dtype, int b_parts, long long b_stride, const void* wb, float inner_eps,
                                float factor, const void* wp, int center_p, float eps_p, const void* w, float offset, int center,
                                float eps, int w_dtype, void* out, int out_dtype, const int* rows, int n, int H,
                                cudaStream_t stream) {
    if (w == nullptr) return WLLM_BAD_SIZE;
    return wllm_sandwich_norm_offset(resid, a, a_dtype, a_parts, a_stride, wa, b, b_dtype, b_parts, b_stride, wb, inner_eps, factor,
                                     wp, 0.f, center_p, eps_p, w, offset, center, eps, w_dtype, out, out_dtype, rows, n, H, stream);
}
