// Rotary position encoding of the query and key heads of a fused q|k|v row, and the write of the
// rotated keys and the values into the pages of the cache.
//
//   angle = float(position) * inv_freq[j],  j < rot_dim/2        (32-bit, sinf/cosf)
//   y[j]         = x[j] * cos - x[j + rot/2] * sin
//   y[j + rot/2] = x[j + rot/2] * cos + x[j] * sin                (pairs j, j + rot/2)
// or, with `interleaved`, the same rotation of the pairs (2j, 2j + 1).
// Dimensions from rot_dim up to head_dim pass through unrotated.  The rotated queries go to `q_out`
// [n, nq * hd].  The input row may come as `in_splits` partial sums (slabs `in_split_stride` elements
// apart, as the split-K matrix product leaves them), which are added in slab order first.  A token
// whose slot is negative writes nothing to the cache (a layer that reads another layer's cache); with nkv = 0 and no
// slots the row holds query heads alone.
// Value heads may have a size of their own (`vd`): the fused row is nq heads of hd, nkv heads of hd, nkv heads
// of vd.  With `unit_norm` every rotated query and key head is divided by its root mean square,
// y / sqrt(mean(y^2) + norm_eps), in 32-bit, before it is rounded and stored.
//
// With row gains (`wllm_rope_row_norm_kv_write`) the query row and the key row of a token are normed as wholes, all heads at
// once, in front of the turn: q <- q / sqrt(mean(q^2) + eps) * wq over the token's nq * hd query elements, the same for k.
// There the projections may have a bias (one 32-bit row for q | k | v, added to the finished sums, in front of the norms), and
// the values may be blended with an earlier layer's values of the same token before they are cached.
//
// Page layout: [page][kv_head][slot_in_page][head_dim] (values: [..][vd]); `slots[n]` is page * page_size + slot_in_page.
#include "common.cuh"

// Two launch shapes.  Fewer than 1,024 tokens (a decode step, a short prompt): grid (token, head), so that the heads of a token run on
// different SMs; head < nq rotates a query head into q_out, nq <= head < nq + nkv rotates a key head into
// its page, the rest copy a value head into its page.  Many tokens: one CTA a token (ALL_HEADS), which
// computes the sines and cosines of the token's position once and walks the heads with them.
// Positions, slots and frequencies are written by no kernel of the step: the angles are worked out before
// the kernel waits for the product it rotates.
template <typename TI, typename TO, bool ALL_HEADS>
__global__ void rope_kv_write_kernel(const TI* __restrict__ qkv, int row_stride, int in_splits, size_t in_split_stride,
                                     TO* __restrict__ q_out, int q_stride, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const float* __restrict__ inv_freq,
                                     TO* __restrict__ k_pages, TO* __restrict__ v_pages, int nq, int nkv, int hd,
                                     int rot_dim, int page_size, int interleaved, int vd) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    // the angle of this thread's first pair (all of them when the block is as wide as half the rotary size)
    float s0 = 0.f, c0 = 1.f;
    if ((int)threadIdx.x < half) sincosf(pos * inv_freq[threadIdx.x], &s0, &c0);
    pdl_wait();
    const int h_lo = ALL_HEADS ? 0 : blockIdx.y, h_hi = ALL_HEADS ? nq + 2 * nkv : blockIdx.y + 1;
    for (int h = h_lo; h < h_hi; ++h) {
        const bool value = h >= nq + nkv;
        const TI* x = qkv + (size_t)t * row_stride + (value ? (size_t)(nq + nkv) * hd + (size_t)(h - nq - nkv) * vd : (size_t)h * hd);
        TO* dst;
        if (h < nq) {
            dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
        } else {
            if (slot < 0) break;
            const int kvh = value ? h - nq - nkv : h - nq;
            TO* pages = value ? v_pages : k_pages;
            dst = pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * (value ? vd : hd);
        }
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
        if (value) {
            for (int c = threadIdx.x; c < vd; c += blockDim.x) dst[c] = from_f32<TO>(in(c));
            continue;
        }
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float sn = s0, cs = c0;
            if (j != (int)threadIdx.x) sincosf(pos * inv_freq[j], &sn, &cs);
            const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
            const float x1 = in(ia), x2 = in(ib);
            float y1, y2;
            rotate_pair(x1, x2, sn, cs, y1, y2);
            dst[ia] = from_f32<TO>(y1);
            dst[ib] = from_f32<TO>(y2);
        }
        for (int c = rot_dim + threadIdx.x; c < hd; c += blockDim.x) dst[c] = from_f32<TO>(in(c));
    }
}

// Heads that are divided by their root mean square after the turn: a warp a head (grid (token, groups of heads)),
// the head's elements in the lanes' registers between the turn and the scaling, the sum of squares by shuffles: no
// barrier, no shared memory, and the same arithmetic for a head whatever the step's size.  Value heads are copied.
// Head sizes up to 512, rotary sizes up to 512.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
rope_unit_norm_kernel(const TI* __restrict__ qkv, int row_stride, int in_splits, size_t in_split_stride,
                      TO* __restrict__ q_out, int q_stride, const int* __restrict__ positions,
                      const int* __restrict__ slots, const float* __restrict__ inv_freq,
                      TO* __restrict__ k_pages, TO* __restrict__ v_pages, int nq, int nkv, int hd,
                      int rot_dim, int page_size, int interleaved, int vd, float norm_eps) {
    pdl_launch_dependents();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);       // this warp's head
    if (h >= nq + 2 * nkv) return;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    float sn[8], cs[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        sn[u] = 0.f; cs[u] = 1.f;
        const int j = lane + 32 * u;
        if (j < half && h < nq + nkv) sincosf(pos * inv_freq[j], &sn[u], &cs[u]);
    }
    pdl_wait();
    {
        const bool value = h >= nq + nkv;
        if (h >= nq && slot < 0) return;
        const TI* x = qkv + (size_t)t * row_stride + (value ? (size_t)(nq + nkv) * hd + (size_t)(h - nq - nkv) * vd : (size_t)h * hd);
        TO* dst;
        if (h < nq) dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
        else {
            const int kvh = value ? h - nq - nkv : h - nq;
            dst = (value ? v_pages : k_pages) + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * (value ? vd : hd);
        }
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
        if (value) {
            for (int c = lane; c < vd; c += 32) dst[c] = from_f32<TO>(in(c));
            return;
        }
        float ya[8], yb[8], yr[16];
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = lane + 32 * u;
            ya[u] = yb[u] = 0.f;
            if (j < half) {
                const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
                rotate_pair(in(ia), in(ib), sn[u], cs[u], ya[u], yb[u]);
                ss += ya[u] * ya[u] + yb[u] * yb[u];
            }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int c = rot_dim + lane + 32 * u;
            yr[u] = 0.f;
            if (c < hd) { yr[u] = in(c); ss += yr[u] * yr[u]; }
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hd + norm_eps);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = lane + 32 * u;
            if (j < half) {
                const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
                dst[ia] = from_f32<TO>(ya[u] * inv);
                dst[ib] = from_f32<TO>(yb[u] * inv);
            }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int c = rot_dim + lane + 32 * u;
            if (c < hd) dst[c] = from_f32<TO>(yr[u] * inv);
        }
    }
}

// The same for prompts in bfloat16 (one input tensor, head sizes, half the rotary size and what lies behind it in steps of 8,
// aligned rows): a CTA a token; the token's sines and cosines go to shared memory once; a warp takes every fourth head, a
// lane eight neighbouring pairs (or eight of the elements behind them) with 16-byte loads and stores; value heads are
// copied sixteen bytes at a time.  Head sizes up to 512.
__global__ void __launch_bounds__(128)
rope_unit_norm_rows_kernel(const bf16* __restrict__ qkv, int row_stride, bf16* __restrict__ q_out, int q_stride,
                           const int* __restrict__ positions, const int* __restrict__ slots, const float* __restrict__ inv_freq,
                           bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int nq, int nkv, int hd, int rot_dim,
                           int page_size, int vd, float norm_eps) {
    extern __shared__ float sc[];            // [half] sines, [half] cosines
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sc[j], &sc[half + j]);
    __syncthreads();
    pdl_wait();
    const bf16* row = qkv + (size_t)t * row_stride;
    const int rotated = slot < 0 ? nq : nq + nkv;
    const int pair_items = half / 8, rest_items = (hd - rot_dim) / 8;       // at most 32 and 64
    for (int h = warp; h < rotated; h += 4) {
        const bf16* x = row + (size_t)h * hd;
        bf16* dst = h < nq ? q_out + (size_t)t * q_stride + (size_t)h * hd
                           : k_pages + (((size_t)(slot / page_size) * nkv + (h - nq)) * page_size + slot % page_size) * hd;
        float ya[8], yb[8], yr[2][8];
        float ss = 0.f;
        if (lane < pair_items) {
            const int j = lane * 8;
            const uint4 a = *reinterpret_cast<const uint4*>(x + j), b = *reinterpret_cast<const uint4*>(x + j + half);
            const bf16* xa = reinterpret_cast<const bf16*>(&a);
            const bf16* xb = reinterpret_cast<const bf16*>(&b);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                rotate_pair(to_f32(xa[e]), to_f32(xb[e]), sc[j + e], sc[half + j + e], ya[e], yb[e]);
                ss += ya[e] * ya[e] + yb[e] * yb[e];
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int item = lane + 32 * u;
            if (item < rest_items) {
                const uint4 r = *reinterpret_cast<const uint4*>(x + rot_dim + item * 8);
                const bf16* xr = reinterpret_cast<const bf16*>(&r);
#pragma unroll
                for (int e = 0; e < 8; ++e) { yr[u][e] = to_f32(xr[e]); ss += yr[u][e] * yr[u][e]; }
            }
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hd + norm_eps);
        if (lane < pair_items) {
            uint4 oa, ob;
            bf16* pa = reinterpret_cast<bf16*>(&oa);
            bf16* pb = reinterpret_cast<bf16*>(&ob);
#pragma unroll
            for (int e = 0; e < 8; ++e) { pa[e] = from_f32<bf16>(ya[e] * inv); pb[e] = from_f32<bf16>(yb[e] * inv); }
            *reinterpret_cast<uint4*>(dst + lane * 8) = oa;
            *reinterpret_cast<uint4*>(dst + lane * 8 + half) = ob;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int item = lane + 32 * u;
            if (item < rest_items) {
                uint4 o;
                bf16* po = reinterpret_cast<bf16*>(&o);
#pragma unroll
                for (int e = 0; e < 8; ++e) po[e] = from_f32<bf16>(yr[u][e] * inv);
                *reinterpret_cast<uint4*>(dst + rot_dim + item * 8) = o;
            }
        }
    }
    if (slot < 0) return;
    const int whole = vd / 8;
    for (int item = threadIdx.x; item < nkv * whole; item += blockDim.x) {
        const int kvh = item / whole, c = (item % whole) * 8;
        bf16* dst = v_pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * vd;
        *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(row + (size_t)(nq + nkv) * hd + (size_t)kvh * vd + c);
    }
}

// Many tokens, bfloat16 in and out, one input tensor, head size and half the rotary size in steps of 8: one
// CTA a token; the token's sines and cosines go to shared memory once; every thread then takes eight
// neighbouring pairs of one head with 16-byte loads and stores, so that a block of 128 threads has the heads
// of a Gemma-2B token in flight at once.  The arithmetic per element is that of the kernel above.
__global__ void rope_kv_write_rows_kernel(const bf16* __restrict__ qkv, int row_stride, bf16* __restrict__ q_out, int q_stride,
                                          const int* __restrict__ positions, const int* __restrict__ slots,
                                          const float* __restrict__ inv_freq, bf16* __restrict__ k_pages,
                                          bf16* __restrict__ v_pages, int nq, int nkv, int hd, int rot_dim, int page_size,
                                          int interleaved) {
    extern __shared__ float sc[];            // [half] sines, [half] cosines
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sc[j], &sc[half + j]);
    __syncthreads();
    pdl_wait();
    const bf16* row = qkv + (size_t)t * row_stride;
    auto dst_of = [&](int h) -> bf16* {
        if (h < nq) return q_out + (size_t)t * q_stride + (size_t)h * hd;
        const int kvh = h < nq + nkv ? h - nq : h - nq - nkv;
        bf16* pages = h < nq + nkv ? k_pages : v_pages;
        return pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * hd;
    };
    const int heads = slot < 0 ? nq : nq + 2 * nkv;
    // rotated heads: items of eight pairs (j .. j + 7 and their partners)
    const int per_head = half / 8, rotated = min(heads, nq + nkv);
    for (int item = threadIdx.x; item < rotated * per_head; item += blockDim.x) {
        const int h = item / per_head, j = (item % per_head) * 8;
        const bf16* x = row + (size_t)h * hd;
        if (interleaved) {          // the pairs (2j, 2j+1) .. (2j+14, 2j+15): sixteen neighbouring elements
            const uint4 a = *reinterpret_cast<const uint4*>(x + 2 * j), b = *reinterpret_cast<const uint4*>(x + 2 * j + 8);
            const bf16* xa = reinterpret_cast<const bf16*>(&a);
            const bf16* xb = reinterpret_cast<const bf16*>(&b);
            uint4 ya, yb;
            bf16* pa = reinterpret_cast<bf16*>(&ya);
            bf16* pb = reinterpret_cast<bf16*>(&yb);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const bf16* src = e < 4 ? xa : xb;
                bf16* to = e < 4 ? pa : pb;
                const int o = (e & 3) * 2;
                float y1, y2;
                rotate_pair(to_f32(src[o]), to_f32(src[o + 1]), sc[j + e], sc[half + j + e], y1, y2);
                to[o] = from_f32<bf16>(y1);
                to[o + 1] = from_f32<bf16>(y2);
            }
            bf16* dst = dst_of(h);
            *reinterpret_cast<uint4*>(dst + 2 * j) = ya;
            *reinterpret_cast<uint4*>(dst + 2 * j + 8) = yb;
            continue;
        }
        const uint4 a = *reinterpret_cast<const uint4*>(x + j), b = *reinterpret_cast<const uint4*>(x + j + half);
        const bf16* xa = reinterpret_cast<const bf16*>(&a);
        const bf16* xb = reinterpret_cast<const bf16*>(&b);
        uint4 ya, yb;
        bf16* pa = reinterpret_cast<bf16*>(&ya);
        bf16* pb = reinterpret_cast<bf16*>(&yb);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float x1 = to_f32(xa[e]), x2 = to_f32(xb[e]), sn = sc[j + e], cs = sc[half + j + e];
            float y1, y2;
            rotate_pair(x1, x2, sn, cs, y1, y2);
            pa[e] = from_f32<bf16>(y1);
            pb[e] = from_f32<bf16>(y2);
        }
        bf16* dst = dst_of(h);
        *reinterpret_cast<uint4*>(dst + j) = ya;
        *reinterpret_cast<uint4*>(dst + j + half) = yb;
    }
    // what is not rotated: the tails of the rotated heads and the value heads, eight elements at a time
    const int tail = (hd - rot_dim) / 8, whole = hd / 8;
    const int copies = rotated * tail + (heads - rotated) * whole;
    for (int item = threadIdx.x; item < copies; item += blockDim.x) {
        int h, c;
        if (item < rotated * tail) { h = item / tail; c = rot_dim + (item % tail) * 8; }
        else { const int v = item - rotated * tail; h = rotated + v / whole; c = (v % whole) * 8; }
        *reinterpret_cast<uint4*>(dst_of(h) + c) = *reinterpret_cast<const uint4*>(row + (size_t)h * hd + c);
    }
}

// The query row and the key row of a token normed as wholes in front of the turn.  One CTA a token: the row's q and k parts
// (partial sums added in slab order) go to shared memory with their sums of squares (block sums in a fixed order, so a
// token's result does not depend on the step), then every thread turns pairs of the normed, gained elements.  The means
// divide by q_count and k_count (heads that are held in steps of 8 elements carry zeros behind them, which count for nothing).
__device__ __forceinline__ float gain_at(const void* p, int dtype, int i) {
    return dtype == WLLM_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
rope_row_norm_kernel(const TI* __restrict__ qkv, int row_stride, int in_splits, size_t in_split_stride,
                     TO* __restrict__ q_out, int q_stride, const int* __restrict__ positions,
                     const int* __restrict__ slots, const float* __restrict__ inv_freq,
                     TO* __restrict__ k_pages, TO* __restrict__ v_pages, int nq, int nkv, int hd,
                     int rot_dim, int page_size, int interleaved, int vd, const void* __restrict__ wq,
                     const void* __restrict__ wk, int w_dtype, int q_count, int k_count, float eps,
                     const float* __restrict__ bias, float* __restrict__ v_first, const float* __restrict__ lam, int mix_mode) {
    extern __shared__ float row[];            // [(nq + nkv) * hd] the token's q and k parts, [half] sines, [half] cosines
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1, qw = nq * hd, kw = nkv * hd;
    float* sn = row + qw + kw;
    float* cs = sn + half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
    pdl_wait();
    const TI* x = qkv + (size_t)t * row_stride;
    auto sum_in = [&](int c) {     // part 0 + part 1 + ... in order; sixteen loads are in flight at a time
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
    auto in = [&](int c) { return bias ? sum_in(c) + bias[c] : sum_in(c); };      // the projection's bias joins the finished sum
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x; c < qw + kw; c += blockDim.x) {
        const float v = in(c);
        row[c] = v;
        if (c < qw) ssq += v * v; else ssk += v * v;
    }
    ssq = block_sum(ssq, scratch);
    ssk = block_sum(ssk, scratch);
    const float inv_q = 1.0f / sqrtf(ssq / (float)q_count + eps);
    const float inv_k = kw > 0 ? 1.0f / sqrtf(ssk / (float)k_count + eps) : 0.f;
    const int heads = slot < 0 ? nq : nq + nkv;
    auto dst_of = [&](int h) -> TO* {
        if (h < nq) return q_out + (size_t)t * q_stride + (size_t)h * hd;
        return k_pages + (((size_t)(slot / page_size) * nkv + (h - nq)) * page_size + slot % page_size) * hd;
    };
    auto normed = [&](int h, int c) {     // element c of head h, normed and gained
        return h < nq ? (row[h * hd + c] * inv_q) * gain_at(wq, w_dtype, h * hd + c)
                      : (row[h * hd + c] * inv_k) * gain_at(wk, w_dtype, (h - nq) * hd + c);
    };
    for (int item = threadIdx.x; item < heads * half; item += blockDim.x) {
        const int h = item / half, j = item % half;
        const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
        float y1, y2;
        rotate_pair(normed(h, ia), normed(h, ib), sn[j], cs[j], y1, y2);
        TO* dst = dst_of(h);
        dst[ia] = from_f32<TO>(y1);
        dst[ib] = from_f32<TO>(y2);
    }
    const int rest = hd - rot_dim;
    for (int item = threadIdx.x; item < heads * rest; item += blockDim.x) {
        const int h = item / rest, c = rot_dim + item % rest;
        dst_of(h)[c] = from_f32<TO>(normed(h, c));
    }
    if (slot < 0) return;
    // mix_mode 1: the token's values are left in v_first [n, nkv * vd] for the layers behind this one; 2: the cached values
    // are (1 - lam) v + lam v_first, in 32-bit, rounded once
    const float l = mix_mode == 2 ? lam[0] : 0.f;
    for (int item = threadIdx.x; item < nkv * vd; item += blockDim.x) {
        const int kvh = item / vd, c = item % vd;
        float v = in(qw + kw + item);
        if (mix_mode == 1) v_first[(size_t)t * nkv * vd + item] = v;
        else if (mix_mode == 2) v = fmaf(l, v_first[(size_t)t * nkv * vd + item], (1.0f - l) * v);
        v_pages[(((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * vd + c] = from_f32<TO>(v);
    }
}

// The same for bfloat16 rows and gains whose heads, turned part and pitches come in steps of 8 elements: 16-byte loads and
// stores, eight neighbouring elements a thread.  An element's partner is read from the row in shared memory, and the two
// products of a turn are rounded apart as in rotate_pair, so an element gets the bits that the kernel above gives it
// from the same sums of squares (the sums themselves are added up in another order here; a model always runs one of the two).
__global__ void __launch_bounds__(256)
rope_row_norm_vec_kernel(const bf16* __restrict__ qkv, int row_stride, bf16* __restrict__ q_out, int q_stride,
                         const int* __restrict__ positions, const int* __restrict__ slots, const float* __restrict__ inv_freq,
                         bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int nq, int nkv, int hd, int rot_dim,
                         int page_size, int interleaved, int vd, const bf16* __restrict__ wq, const bf16* __restrict__ wk,
                         int q_count, int k_count, float eps, const float* __restrict__ bias, float* __restrict__ v_first,
                         const float* __restrict__ lam, int mix_mode) {
    extern __shared__ float row[];            // [(nq + nkv) * hd] the token's q and k parts, [half] sines, [half] cosines
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1, qw = nq * hd, kw = nkv * hd;
    float* sn = row + qw + kw;
    float* cs = sn + half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
    pdl_wait();
    const bf16* x = qkv + (size_t)t * row_stride;
    float ssq = 0.f, ssk = 0.f;
    for (int c0 = threadIdx.x * 8; c0 < qw + kw; c0 += blockDim.x * 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + c0);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 v = __bfloat1622float2(p2[e]);
            if (bias) { v.x += bias[c0 + 2 * e]; v.y += bias[c0 + 2 * e + 1]; }      // the projection's bias joins the finished sum
            row[c0 + 2 * e] = v.x; row[c0 + 2 * e + 1] = v.y;
            ss += v.x * v.x; ss += v.y * v.y;
        }
        if (c0 < qw) ssq += ss; else ssk += ss;          // qw is a multiple of 8: a chunk lies on one side
    }
    ssq = block_sum(ssq, scratch);
    ssk = block_sum(ssk, scratch);
    const float inv_q = 1.0f / sqrtf(ssq / (float)q_count + eps);
    const float inv_k = kw > 0 ? 1.0f / sqrtf(ssk / (float)k_count + eps) : 0.f;
    const int heads = slot < 0 ? nq : nq + nkv, per_head = hd >> 3;
    for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
        const int h = item / per_head, c0 = (item % per_head) * 8;
        const bool is_q = h < nq;
        const float inv = is_q ? inv_q : inv_k;
        const bf16* gain = is_q ? wq + h * hd : wk + (h - nq) * hd;
        const float* src = row + h * hd;
        const uint4 graw = *reinterpret_cast<const uint4*>(gain + c0);
        const bf16* g8 = reinterpret_cast<const bf16*>(&graw);
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int c = c0 + e;
            const float mine = (src[c] * inv) * __bfloat162float(g8[e]);
            y[e] = mine;
            if (c < rot_dim) {
                const bool first = interleaved ? !(c & 1) : c < half;
                const int j = interleaved ? c >> 1 : (first ? c : c - half);
                const int pc = interleaved ? c ^ 1 : (first ? c + half : c - half);
                const float other = (src[pc] * inv) * __bfloat162float(gain[pc]);
                const float a = __fmul_rn(mine, cs[j]), b = __fmul_rn(other, sn[j]);
                y[e] = first ? __fsub_rn(a, b) : __fadd_rn(a, b);
            }
        }
        uint4 packed;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(y[2 * e], y[2 * e + 1]);
        bf16* dst = is_q ? q_out + (size_t)t * q_stride + (size_t)h * hd
                         : k_pages + (((size_t)(slot / page_size) * nkv + (h - nq)) * page_size + slot % page_size) * hd;
        *reinterpret_cast<uint4*>(dst + c0) = packed;
    }
    if (slot < 0) return;
    const int v_per = vd >> 3;
    const float l = mix_mode == 2 ? lam[0] : 0.f;
    for (int item = threadIdx.x; item < nkv * v_per; item += blockDim.x) {
        const int kvh = item / v_per, c0 = (item % v_per) * 8;
        uint4 raw = *reinterpret_cast<const uint4*>(x + qw + kw + kvh * vd + c0);
        if (bias != nullptr || mix_mode != 0) {
            // as in the kernel above: the bias, then the values left for later layers (unrounded) or blended with an earlier layer's
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
            float* keep = v_first + (size_t)t * nkv * vd + kvh * vd + c0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 v = __bfloat1622float2(h2[e]);
                if (bias) { v.x += bias[qw + kw + kvh * vd + c0 + 2 * e]; v.y += bias[qw + kw + kvh * vd + c0 + 2 * e + 1]; }
                if (mix_mode == 1) { keep[2 * e] = v.x; keep[2 * e + 1] = v.y; }
                else if (mix_mode == 2) { v.x = fmaf(l, keep[2 * e], (1.0f - l) * v.x); v.y = fmaf(l, keep[2 * e + 1], (1.0f - l) * v.y); }
                h2[e] = __floats2bfloat162_rn(v.x, v.y);
            }
        }
        *reinterpret_cast<uint4*>(v_pages + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * vd + c0) = raw;
    }
}

// wq [nq * hd], wk [nkv * hd]: the gains of the two row norms (one element type); q_count, k_count: the elements that
// count for the means (nq * hd and nkv * hd unless the heads are held with zeros behind them).
WLLM_API int wllm_rope_row_norm_kv_write(const void* qkv, int in_dtype, int row_stride, int in_splits, long long in_split_stride,
                                         void* q_out, int out_dtype, int q_stride, const int* positions, const int* slots,
                                         const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                         int rot_dim, int page_size, int interleaved, int vd, const void* wq, const void* wk,
                                         int w_dtype, int q_count, int k_count, float eps, const float* bias, float* v_first,
                                         const float* lam, int mix_mode, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (mix_mode < 0 || mix_mode > 2 || (mix_mode > 0 && (v_first == nullptr || slots == nullptr)) || (mix_mode == 2 && lam == nullptr))
        return WLLM_BAD_SIZE;
    if (hd <= 0 || vd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || page_size <= 0 || nq <= 0 || nkv < 0 ||
        (nkv == 0 && slots != nullptr) || in_splits < 1 || q_count <= 0 || (nkv > 0 && k_count <= 0) || wq == nullptr ||
        (nkv > 0 && wk == nullptr))
        return WLLM_BAD_SIZE;
    if (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32) return WLLM_BAD_DTYPE;
    const size_t smem = ((size_t)(nq + nkv) * hd + rot_dim) * sizeof(float);
    if (smem > 200 * 1024) return WLLM_BAD_SIZE;
#define RN(TI, TO) do { \
        static bool raised = false; \
        if (!raised && smem > 48 * 1024) { \
            const cudaError_t e = cudaFuncSetAttribute(rope_row_norm_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return 1000 + (int)e; \
            raised = true; \
        } \
        return wllm_launch(rope_row_norm_kernel<TI, TO>, n, 256, smem, stream, (const TI*)qkv, row_stride, in_splits, \
            (size_t)in_split_stride, (TO*)q_out, q_stride, positions, slots, inv_freq, (TO*)k_pages, (TO*)v_pages, nq, nkv, hd, \
            rot_dim, page_size, interleaved, vd, wq, wk, w_dtype, q_count, k_count, eps, bias, v_first, lam, mix_mode); \
    } while (0)
    const bool aligned = !(((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)wq | (uintptr_t)wk) & 15);
    if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16 && w_dtype == WLLM_BF16 && in_splits == 1 && aligned && hd % 8 == 0 &&
        vd % 8 == 0 && rot_dim % 8 == 0 && row_stride % 8 == 0 && q_stride % 8 == 0) {
        static bool raised = false;
        if (!raised && smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(rope_row_norm_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return 1000 + (int)e;
            raised = true;
        }
        return wllm_launch(rope_row_norm_vec_kernel, n, 256, smem, stream, (const bf16*)qkv, row_stride, (bf16*)q_out, q_stride,
                           positions, slots, inv_freq, (bf16*)k_pages, (bf16*)v_pages, nq, nkv, hd, rot_dim, page_size, interleaved,
                           vd, (const bf16*)wq, (const bf16*)wk, q_count, k_count, eps, bias, v_first, lam, mix_mode);
    }
    if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16) RN(bf16, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_BF16) RN(float, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_F32) RN(float, float);
#undef RN
    return WLLM_BAD_DTYPE;
}

// vd: size of a value head (hd when they are the same); unit_norm: divide rotated q and k heads by their root mean square.
WLLM_API int wllm_rope_kv_write_general(const void* qkv, int in_dtype, int row_stride, int in_splits, long long in_split_stride,
                                        void* q_out, int out_dtype, int q_stride, const int* positions, const int* slots,
                                        const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                        int rot_dim, int page_size, int interleaved, int vd, int unit_norm, float norm_eps,
                                        cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (hd <= 0 || vd <= 0 || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || page_size <= 0 || nq <= 0 || nkv < 0 || (nkv == 0 && slots != nullptr) || in_splits < 1)
        return WLLM_BAD_SIZE;
    if (n >= 256 && vd == hd && !unit_norm && in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16 && in_splits == 1 && hd % 8 == 0 && rot_dim % 16 == 0 &&
        row_stride % 8 == 0 && q_stride % 8 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) &&
        !((uintptr_t)k_pages & 15) && !((uintptr_t)v_pages & 15))
        return wllm_launch(rope_kv_write_rows_kernel, n, 128, (size_t)rot_dim * sizeof(float), stream, (const bf16*)qkv, row_stride,
                           (bf16*)q_out, q_stride, positions, slots, inv_freq, (bf16*)k_pages, (bf16*)v_pages, nq, nkv, hd,
                           rot_dim, page_size, interleaved);
    if (unit_norm) {
        if (hd > 512) return WLLM_BAD_SIZE;
        if (n >= 256 && !interleaved && in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16 && in_splits == 1 && hd % 8 == 0 && vd % 8 == 0 &&
            rot_dim % 16 == 0 && row_stride % 8 == 0 && q_stride % 8 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) &&
            !((uintptr_t)k_pages & 15) && !((uintptr_t)v_pages & 15))
            return wllm_launch(rope_unit_norm_rows_kernel, n, 128, (size_t)rot_dim * sizeof(float), stream, (const bf16*)qkv, row_stride,
                               (bf16*)q_out, q_stride, positions, slots, inv_freq, (bf16*)k_pages, (bf16*)v_pages, nq, nkv, hd,
                               rot_dim, page_size, vd, norm_eps);
        // four heads a CTA at every size.  A CTA a token whose warps walk every fourth head (angles worked out once a lane)
        // was measured slower over a prompt: 2,048 tokens, 10 heads of 256: 76 us against 48
        const dim3 ugrid(n, (nq + 2 * nkv + 3) / 4);
#define UN(TI, TO) wllm_launch(rope_unit_norm_kernel<TI, TO>, ugrid, 128, 0, stream, (const TI*)qkv, row_stride, in_splits, \
        (size_t)in_split_stride, (TO*)q_out, q_stride, positions, slots, inv_freq, (TO*)k_pages, (TO*)v_pages, nq, nkv, hd, \
        rot_dim, page_size, interleaved, vd, norm_eps)
        if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16) return UN(bf16, bf16);
        if (in_dtype == WLLM_F32 && out_dtype == WLLM_BF16) return UN(float, bf16);
        if (in_dtype == WLLM_F32 && out_dtype == WLLM_F32) return UN(float, float);
#undef UN
        return WLLM_BAD_DTYPE;
    }
    const int threads = hd >= 256 ? 128 : (hd >= 128 ? 64 : 32);
    // One CTA a token once the tokens alone fill the SMs several times over; below that a CTA a head, which keeps a
    // token's heads (and the partial sums each has to add) on different SMs: 256 tokens x 10 heads of 4 parts took
    // 24 us a layer as 256 CTAs and take 6 as 2,560.
    const bool all_heads = n >= 1024;
    const dim3 grid(n, all_heads ? 1 : nq + 2 * nkv);
#define GO2(TI, TO, A) wllm_launch(rope_kv_write_kernel<TI, TO, A>, grid, threads, 0, stream, (const TI*)qkv, row_stride, in_splits, \
        (size_t)in_split_stride, (TO*)q_out, q_stride, positions, slots, inv_freq, (TO*)k_pages, (TO*)v_pages, nq, nkv, hd, \
        rot_dim, page_size, interleaved, vd)
#define GO(TI, TO) (all_heads ? GO2(TI, TO, true) : GO2(TI, TO, false))
    if (in_dtype == WLLM_BF16 && out_dtype == WLLM_BF16) return GO(bf16, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_BF16) return GO(float, bf16);
    if (in_dtype == WLLM_F32 && out_dtype == WLLM_F32) return GO(float, float);
#undef GO
#undef GO2
    return WLLM_BAD_DTYPE;
}

WLLM_API int wllm_rope_kv_write(const void* qkv, int in_dtype, int row_stride, int in_splits, long long in_split_stride,
                                void* q_out, int out_dtype, int q_stride, const int* positions, const int* slots,
                                const float* inv_freq, void* k_pages, void* v_pages, int n, int nq, int nkv, int hd,
                                int rot_dim, int page_size, int interleaved, cudaStream_t stream) {
    return wllm_rope_kv_write_general(qkv, in_dtype, row_stride, in_splits, in_split_stride, q_out, out_dtype, q_stride,
                                      positions, slots, inv_freq, k_pages, v_pages, n, nq, nkv, hd, rot_dim, page_size,
                                      interleaved, hd, 0, 0.f, stream);
}
