// The gated delta rule: a matrix state per (request, head) that every token first decays, then corrects towards its value
// along its key, then reads with its query:
//
//     S <- g_t S;    u_t = beta_t (v_t - S^T k_t);    S <- S + k_t u_t^T;    o_t = S^T q_t        S: [dim, vdim], 32-bit
//
// g_t in (0, 1) is one decay per head and token, beta_t in (0, 1) one step size per head and token.  q, k and v are each
// filtered along the sequence, channel by channel, by `taps` taps that look back only (the last tap weighs the token itself,
// inputs in front of the sequence count as zero) and pass SiLU; q and k are then scaled to unit length head by head.  Query and key heads may be
// fewer than value heads (head h reads q/k head h / (H / G)).  The state and the convolutions' last taps - 1 inputs live in
// the cache manager's state slots and are carried from step to step, so a whole prompt, a portion and a single decoded token
// are one case and give the same bits.
//
//   wllm_delta_prepare      from a fused projection row (q | k | v | ... | b | a in one matrix product, possibly still in split-K
//                           slabs): convolution and SiLU of q, k and v, the unit norms x / sqrt(sum(x^2) + eps) (q also times
//                           q_scale), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)), all 32-bit.  A warp a head.
//   wllm_delta_conv_update  the slots' last taps - 1 inputs after this step's tokens (a thread a channel, read first, written after).
//   wllm_delta_scan         the recurrence.  The columns of S do not meet: column j needs S[:, j] alone.  Eight or sixteen lanes
//                           hold a column (runs of four key channels each), a CTA of eight warps 32 or 16 columns of one
//                           (request, head); tokens arrive in tiles through a cp.async ring and are walked in order.  With
//                           a = S^T k and b = S^T q taken from the decayed state in one pass (two sums over a column's lanes),
//                           u = beta (v - g a) and o = g b + u (k . q), which is S^T q of the state that already holds the token's update.
#include "common.cuh"

__device__ __forceinline__ float dr_any(const void* p, int dtype, size_t i) {
    return dtype == WLLM_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}
// element i of a row that may come as `parts` 32-bit slabs `stride` elements apart, added in slab order
__device__ __forceinline__ float dr_in(const void* p, int dtype, int parts, size_t stride, size_t i) {
    if (parts == 1) return dr_any(p, dtype, i);
    const float* f = reinterpret_cast<const float*>(p) + i;
    float v = f[0];
    for (int s = 1; s < parts; ++s) v += f[(size_t)s * stride];
    return v;
}
__device__ __forceinline__ float dr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int DR_MAX_TAPS = 16;
constexpr int DR_MAX_PER_LANE = 8;       // key or value channels a lane holds of a head in the prepare kernel: heads up to 256

// grid (tokens, ceil(units / 4)), 128 threads; unit < G: a query head, < 2G: a key head, < 2G + H: a value head, 2G + H: the
// token's beta and decay of every head.
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const void* __restrict__ fused, int in_dtype, int row_stride, int parts, size_t part_stride, int q_off,
                     int k_off, int v_off, int b_off, int a_off, int n, int H, int G, int D, int V, int taps,
                     const void* __restrict__ conv_q, const void* __restrict__ conv_k, const void* __restrict__ conv_v,
                     const void* __restrict__ a_log, const void* __restrict__ dt_bias, int w_dtype,
                     const int* __restrict__ token_req, const int* __restrict__ req_q_start, const int* __restrict__ req_slot,
                     const float* __restrict__ conv_state, float unit_eps, float q_scale, float* __restrict__ q,
                     float* __restrict__ k, float* __restrict__ v, float* __restrict__ beta, float* __restrict__ decay) {
    pdl_begin();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.y * 4 + warp;
    if (unit > 2 * G + H) return;
    if (unit == 2 * G + H) {
        for (int h = lane; h < H; h += 32) {
            const float bz = dr_in(fused, in_dtype, parts, part_stride, (size_t)t * row_stride + b_off + h);
            const float az = dr_in(fused, in_dtype, parts, part_stride, (size_t)t * row_stride + a_off + h);
            beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-bz));
            decay[(size_t)t * H + h] = expf(-expf(dr_any(a_log, w_dtype, h)) * dr_softplus(az + dr_any(dt_bias, w_dtype, h)));
        }
        return;
    }
    const int r = token_req[t];
    const int i = t - req_q_start[r], slot = req_slot[r];       // the token's place in its request's portion
    const int C = 2 * G * D + H * V;
    int col0, chan0, size, head;
    const void* w;
    if (unit < G) { head = unit; size = D; col0 = q_off + head * D; chan0 = head * D; w = conv_q; }
    else if (unit < 2 * G) { head = unit - G; size = D; col0 = k_off + head * D; chan0 = G * D + head * D; w = conv_k; }
    else { head = unit - 2 * G; size = V; col0 = v_off + head * V; chan0 = 2 * G * D + head * V; w = conv_v; }
    float y[DR_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < DR_MAX_PER_LANE; ++e) {
        const int c = lane + 32 * e;
        y[e] = 0.f;
        if (c < size) {
            float acc = 0.f;
            for (int j = taps - 1; j >= 0; --j) {            // the oldest input first: one order for every way of cutting
                float x;
                if (i - j >= 0) x = dr_in(fused, in_dtype, parts, part_stride, (size_t)(t - j) * row_stride + col0 + c);
                else x = slot >= 0 ? conv_state[((size_t)slot * (taps - 1) + (taps - 1 + i - j)) * C + chan0 + c] : 0.f;
                acc = fmaf(dr_any(w, w_dtype, (size_t)(head * size + c) * taps + (taps - 1 - j)), x, acc);
            }
            y[e] = dr_silu(acc);
            ss = fmaf(y[e], y[e], ss);
        }
    }
    if (unit < 2 * G) {
        ss = warp_sum(ss);
        const float inv = (1.0f / sqrtf(ss + unit_eps)) * (unit < G ? q_scale : 1.0f);
        float* dst = (unit < G ? q : k) + ((size_t)t * G + head) * D;
#pragma unroll
        for (int e = 0; e < DR_MAX_PER_LANE; ++e)
            if (lane + 32 * e < size) dst[lane + 32 * e] = y[e] * inv;
    } else {
        float* dst = v + ((size_t)t * H + head) * V;
#pragma unroll
        for (int e = 0; e < DR_MAX_PER_LANE; ++e)
            if (lane + 32 * e < size) dst[lane + 32 * e] = y[e];
    }
}

// grid (requests, ceil(C / 256)): a thread a channel; the taps - 1 inputs that end at the request's last token of this step
__global__ void __launch_bounds__(256)
delta_conv_update_kernel(const void* __restrict__ fused, int in_dtype, int row_stride, int parts, size_t part_stride, int q_off,
                         int k_off, int v_off, int H, int G, int D, int V, int taps, const int* __restrict__ req_q_start,
                         const int* __restrict__ req_q_len, const int* __restrict__ req_slot, float* __restrict__ conv_state) {
    pdl_begin();
    const int r = blockIdx.x, len = req_q_len[r], slot = req_slot[r];
    if (len <= 0 || slot < 0) return;
    const int C = 2 * G * D + H * V, ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (ch >= C) return;
    const int col = ch < G * D ? q_off + ch : (ch < 2 * G * D ? k_off + ch - G * D : v_off + ch - 2 * G * D);
    const int keep = taps - 1, t0 = req_q_start[r];
    float* st = conv_state + (size_t)slot * keep * C + ch;
    float vals[DR_MAX_TAPS];
#pragma unroll
    for (int s = 0; s < DR_MAX_TAPS; ++s) {
        if (s < keep) {
            const int src = len - keep + s;               // place among this step's tokens; negative: an input kept from before
            vals[s] = src >= 0 ? dr_in(fused, in_dtype, parts, part_stride, (size_t)(t0 + src) * row_stride + col)
                               : st[(size_t)(s + len) * C];
        }
    }
#pragma unroll
    for (int s = 0; s < DR_MAX_TAPS; ++s)
        if (s < keep) st[(size_t)s * C] = vals[s];
}

constexpr int DR_TT = 16;          // tokens of a tile
constexpr int DR_THREADS = 256;    // eight warps; with LPC lanes a column a warp holds 32 / LPC columns, a CTA 256 / LPC

__device__ __forceinline__ void dr_cp4(float* smem_dst, const float* src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_cp16(float* smem_dst, const float* src) {      // both 16-byte aligned
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// One token of the walk for the lane's NE key channels of its column (see the kernel below).
template <int NE, int LPC>
__device__ __forceinline__ void delta_token(float (&S)[NE], const float* __restrict__ kr, const float* __restrict__ qr, int sub, float gt,
                                            float bt, float vt, float kq, float& o) {
    // the lane's channels: 4 sub + 4 LPC j + e (j < NE / 4, e < 4): a column's lanes read runs of 128 contiguous bytes a load
    float kv[NE], a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NE / 4; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + 4 * sub + 4 * LPC * j);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + 4 * sub + 4 * LPC * j);
        kv[4 * j] = k4.x; kv[4 * j + 1] = k4.y; kv[4 * j + 2] = k4.z; kv[4 * j + 3] = k4.w;
        a4[0] = fmaf(S[4 * j], k4.x, a4[0]); a4[1] = fmaf(S[4 * j + 1], k4.y, a4[1]);
        a4[2] = fmaf(S[4 * j + 2], k4.z, a4[2]); a4[3] = fmaf(S[4 * j + 3], k4.w, a4[3]);
        b4[0] = fmaf(S[4 * j], q4.x, b4[0]); b4[1] = fmaf(S[4 * j + 1], q4.y, b4[1]);
        b4[2] = fmaf(S[4 * j + 2], q4.z, b4[2]); b4[3] = fmaf(S[4 * j + 3], q4.w, b4[3]);
    }
    float a = (a4[0] + a4[1]) + (a4[2] + a4[3]), b = (b4[0] + b4[1]) + (b4[2] + b4[3]);
#pragma unroll
    for (int off = 1; off < LPC; off <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    const float u = bt * (vt - gt * a);
#pragma unroll
    for (int i = 0; i < NE; ++i) S[i] = fmaf(kv[i], u, gt * S[i]);
    o = fmaf(u, kq, gt * b);
}

// LPC lanes hold a column, NE key channels each (dim <= LPC * NE, in runs of four).  grid (ceil(V / (256 / LPC)), H, requests),
// 256 threads.  The walk is one dependent chain a token (two sums over a column's lanes, the step, the update); a warp alone on
// its scheduler waits out every link of it, so heads of 64 channels and more spread a column over sixteen lanes: half the
// instructions a warp and token, twice the warps (one warp a scheduler issued a third of the time; profiles/delta_scan_2048.txt).
// Tiles of DR_TT tokens come through a ring of two cp.async stages, so that the
// next tile's rows are on their way while this one is walked; a key's and a query's rows are padded with zeros to 32 NE / 4
// channels in shared memory, so the walk carries no guards.  k . q of a tile's tokens is worked out once a tile by the
// warps together (it is the same for every column).
template <int NE, int LPC, int THREADS>
__global__ void __launch_bounds__(THREADS)
delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                  float* __restrict__ out, const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                  const int* __restrict__ req_slot, int H, int G, int D, int V) {
    constexpr int DP = LPC * NE;                        // channels of a row in shared memory
    constexpr int DR_COLS = THREADS / LPC;              // value columns of the CTA
    extern __shared__ __align__(16) float dr_smem[];    // two stages of [TT][DP] q, [TT][DP] k, [TT][16] v, [TT] beta, [TT] decay; [TT] k.q
    pdl_begin();
    const int r = blockIdx.z, h = blockIdx.y;
    const int len = req_q_len[r], slot = req_slot[r];
    if (len <= 0 || slot < 0) return;                      // a request that brings no token
    const int g = h / (H / G), t0 = req_q_start[r];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & (LPC - 1);
    const int col0 = blockIdx.x * DR_COLS, mine = threadIdx.x / LPC, col = col0 + mine;
    const bool live = col < V;
    constexpr int per_stage = DR_TT * (2 * DP + DR_COLS + 2);
    float* kq = dr_smem + 2 * per_stage;
    const bool wide = (D & 3) == 0 && (V & 3) == 0 && ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0);
    if (D < DP)          // the channels behind the head's own stay zero in both stages
        for (int idx = threadIdx.x; idx < 2 * 2 * DR_TT * (DP - D); idx += blockDim.x) {
            const int row = idx / (DP - D), c = D + idx % (DP - D);
            dr_smem[(row / (2 * DR_TT)) * per_stage + (row % (2 * DR_TT)) * DP + c] = 0.f;
        }
    auto load_tile = [&](int tile, int stage) {
        float* qs = dr_smem + stage * per_stage;
        float* ks = qs + DR_TT * DP;
        float* vs = ks + DR_TT * DP;
        float* bs = vs + DR_TT * DR_COLS;
        float* gs = bs + DR_TT;
        const int first = t0 + tile * DR_TT, count = min(DR_TT, len - tile * DR_TT);
        if (wide) {
            const int per_row = D >> 2;
            for (int idx = threadIdx.x; idx < count * per_row; idx += blockDim.x) {
                const int tt = idx / per_row, c = (idx - tt * per_row) * 4;
                const size_t at = ((size_t)(first + tt) * G + g) * D + c;
                dr_cp16(qs + tt * DP + c, q + at);
                dr_cp16(ks + tt * DP + c, k + at);
            }
            for (int idx = threadIdx.x; idx < count * (DR_COLS / 4); idx += blockDim.x) {
                const int tt = idx / (DR_COLS / 4), cc = (idx % (DR_COLS / 4)) * 4;
                const float* vrow = v + ((size_t)(first + tt) * H + h) * V;
                if (col0 + cc + 3 < V) dr_cp16(vs + tt * DR_COLS + cc, vrow + col0 + cc);
                else
                    for (int e = 0; e < 4; ++e) dr_cp4(vs + tt * DR_COLS + cc + e, vrow + min(col0 + cc + e, V - 1));
            }
        } else {
            for (int idx = threadIdx.x; idx < count * D; idx += blockDim.x) {
                const int tt = idx / D, c = idx - tt * D;
                const size_t at = ((size_t)(first + tt) * G + g) * D + c;
                dr_cp4(qs + tt * DP + c, q + at);
                dr_cp4(ks + tt * DP + c, k + at);
            }
            for (int idx = threadIdx.x; idx < count * DR_COLS; idx += blockDim.x) {
                const int tt = idx / DR_COLS, cc = idx % DR_COLS;
                dr_cp4(vs + idx, v + ((size_t)(first + tt) * H + h) * V + min(col0 + cc, V - 1));
            }
        }
        if (threadIdx.x < count) {
            dr_cp4(bs + threadIdx.x, beta + (size_t)(first + threadIdx.x) * H + h);
            dr_cp4(gs + threadIdx.x, decay + (size_t)(first + threadIdx.x) * H + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float S[NE];
    float* Sg = state + (((size_t)slot * H + h) * D) * V;
#pragma unroll
    for (int i = 0; i < NE; ++i) {
        const int c = 4 * sub + 4 * LPC * (i >> 2) + (i & 3);
        S[i] = (live && c < D) ? Sg[(size_t)c * V + col] : 0.f;
    }
    const int tiles = (len + DR_TT - 1) / DR_TT;
    load_tile(0, 0);
    for (int tile = 0; tile < tiles; ++tile) {
        const int stage = tile & 1;
        if (tile + 1 < tiles) {
            load_tile(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                   // the tile is here for everyone (and the zeros behind the heads, the first time)
        const float* qs = dr_smem + stage * per_stage;
        const float* ks = qs + DR_TT * DP;
        const float* vs = ks + DR_TT * DP;
        const float* bs = vs + DR_TT * DR_COLS;
        const float* gs = bs + DR_TT;
        const int count = min(DR_TT, len - tile * DR_TT);
        for (int tt = warp; tt < count; tt += THREADS / 32) {     // k . q: a lane's strided chain, the warp's tree
            float acc = 0.f;
            for (int c = lane; c < D; c += 32) acc = fmaf(ks[tt * DP + c], qs[tt * DP + c], acc);
            acc = warp_sum(acc);
            if (lane == 0) kq[tt] = acc;
        }
        __syncthreads();
        float* orow = out + ((size_t)(t0 + tile * DR_TT) * H + h) * V + col;
        if (count == DR_TT) {
#pragma unroll 4
            for (int tt = 0; tt < DR_TT; ++tt) {
                float o;
                delta_token<NE, LPC>(S, ks + tt * DP, qs + tt * DP, sub, gs[tt], bs[tt], vs[tt * DR_COLS + mine], kq[tt], o);
                if (live && sub == 0) orow[(size_t)tt * H * V] = o;
            }
        } else {
            for (int tt = 0; tt < count; ++tt) {
                float o;
                delta_token<NE, LPC>(S, ks + tt * DP, qs + tt * DP, sub, gs[tt], bs[tt], vs[tt * DR_COLS + mine], kq[tt], o);
                if (live && sub == 0) orow[(size_t)tt * H * V] = o;
            }
        }
        __syncthreads();                                   // the stage and k . q are read to their end before the next tile overwrites them
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NE; ++i) {
            const int c = 4 * sub + 4 * LPC * (i >> 2) + (i & 3);
            if (c < D) Sg[(size_t)c * V + col] = S[i];
        }
    }
}

// fused [n, W] (or `parts` 32-bit slabs): q at q_off [G * D], k at k_off [G * D], v at v_off [H * V], b at b_off [H], a at a_off [H];
// conv_q, conv_k [G * D, taps], conv_v [H * V, taps], a_log, dt_bias [H] in one element type; conv_state [slots, taps - 1, 2 G D + H V];
// q, k [n, G, D], v [n, H, V], beta, decay [n, H], all 32-bit.
WLLM_API int wllm_delta_prepare(const void* fused, int in_dtype, int row_stride, int parts, long long part_stride, int q_off,
                                int k_off, int v_off, int b_off, int a_off, int n, int H, int G, int D, int V, int taps,
                                const void* conv_q, const void* conv_k, const void* conv_v, const void* a_log, const void* dt_bias,
                                int w_dtype, const int* token_req, const int* req_q_start, const int* req_slot,
                                const float* conv_state, float unit_eps, float q_scale, float* q, float* k, float* v, float* beta,
                                float* decay, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || D > 32 * DR_MAX_PER_LANE || V <= 0 || V > 32 * DR_MAX_PER_LANE || taps < 1 ||
        taps > DR_MAX_TAPS || parts < 1 || (taps > 1 && conv_state == nullptr))
        return WLLM_BAD_SIZE;
    if ((in_dtype != WLLM_BF16 && in_dtype != WLLM_F32) || (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32)) return WLLM_BAD_DTYPE;
    const int units = 2 * G + H + 1;
    if ((units + 3) / 4 > 65535) return WLLM_BAD_SIZE;
    return wllm_launch(delta_prepare_kernel, dim3(n, (units + 3) / 4), 128, 0, stream, fused, in_dtype, row_stride, parts,
                       (size_t)part_stride, q_off, k_off, v_off, b_off, a_off, n, H, G, D, V, taps, conv_q, conv_k, conv_v, a_log,
                       dt_bias, w_dtype, token_req, req_q_start, req_slot, conv_state, unit_eps, q_scale, q, k, v, beta, decay);
}

WLLM_API int wllm_delta_conv_update(const void* fused, int in_dtype, int row_stride, int parts, long long part_stride, int q_off,
                                    int k_off, int v_off, int H, int G, int D, int V, int taps, const int* req_q_start,
                                    const int* req_q_len, const int* req_slot, int requests, float* conv_state, cudaStream_t stream) {
    if (requests <= 0 || taps <= 1) return WLLM_OK;
    if (H <= 0 || G <= 0 || D <= 0 || V <= 0 || taps > DR_MAX_TAPS || parts < 1 || conv_state == nullptr) return WLLM_BAD_SIZE;
    if (in_dtype != WLLM_BF16 && in_dtype != WLLM_F32) return WLLM_BAD_DTYPE;
    const int C = 2 * G * D + H * V;
    if ((C + 255) / 256 > 65535) return WLLM_BAD_SIZE;
    return wllm_launch(delta_conv_update_kernel, dim3(requests, (C + 255) / 256), 256, 0, stream, fused, in_dtype, row_stride, parts,
                       (size_t)part_stride, q_off, k_off, v_off, H, G, D, V, taps, req_q_start, req_q_len, req_slot, conv_state);
}

// state [slots, H, D, V]; out [n, H, V].  Requests by start, length and state slot; a length of 0 or a slot of -1 is passed by.
WLLM_API int wllm_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay, float* state,
                             float* out, const int* req_q_start, const int* req_q_len, const int* req_slot, int requests, int H,
                             int G, int D, int V, cudaStream_t stream) {
    if (requests <= 0) return WLLM_OK;
    if (H <= 0 || H > 65535 || G <= 0 || H % G != 0 || requests > 65535 || D <= 0 || D > 256 || V <= 0) return WLLM_BAD_SIZE;
    // heads of up to 32 channels: eight lanes a column, four channels each; above: sixteen lanes, 4, 8 or 16 channels each
    const int lpc = D <= 32 ? 8 : 16, ne = D <= 64 ? 4 : (D <= 128 ? 8 : 16), threads = DR_THREADS;
    const int cols = threads / lpc;
    const dim3 grid((V + cols - 1) / cols, H, requests);
    const size_t smem = ((size_t)2 * DR_TT * (2 * lpc * ne + cols + 2) + DR_TT) * sizeof(float);
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<16, 16, DR_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return 1000 + (int)e;
        raised = true;
    }
#define SCAN(NE, LPC, TH) wllm_launch(delta_scan_kernel<NE, LPC, TH>, grid, TH, smem, stream, q, k, v, beta, decay, state, out, \
                                      req_q_start, req_q_len, req_slot, H, G, D, V)
    if (D <= 32) return SCAN(4, 8, DR_THREADS);
    if (D <= 64) return SCAN(4, 16, DR_THREADS);
    if (D <= 128) return SCAN(8, 16, DR_THREADS);
    return SCAN(16, 16, DR_THREADS);
#undef SCAN
}
