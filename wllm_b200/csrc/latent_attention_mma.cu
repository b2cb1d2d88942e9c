// bfloat16 attention over cached latent rows on the tensor cores (mma.sync m16n8k16, 32-bit accumulation), compiled
// for one row: -DLATENT_ROW=<elements of a cached row, a multiple of 8> -DLATENT_RANK=<a multiple of 32, <= LATENT_ROW>.
//
// Every query head reads the same cached rows: a row is a key of LATENT_ROW elements whose first LATENT_RANK elements
// are the value as well, so one tile in shared memory serves the scores and the weighted sum.  The rows of a request
// are (token, head) pairs, row m = (token m / heads, head m % heads): all heads of a token share every tile of keys.
//
// One CTA takes 64 rows of one request: eight warps, four groups of 16 rows by two halves of the value's columns.
// Both warps of a pair compute the 16 x 32 scores of their rows (the same numbers, so the same running maximum and
// sum), and each adds its half of the weighted values: an output row of 512 columns would not fit one warp's registers.
// Keys come through the request's block table with 16-byte cp.async into a ring of two swizzled tiles of 32 keys;
// rows outside the keys that the CTA's rows may see are zero-filled.  Scores, maxima, sums and outputs are 32-bit,
// exponentials are exp2 of log2(e)-scaled scores.  window > 0: a row sees itself and the window - 1 keys before it;
// < 0: the earlier keys of its own block of -window positions; 0: every earlier key.
#include "common.cuh"

#if !defined(LATENT_ROW) || !defined(LATENT_RANK)
#error "compile with -DLATENT_ROW=<row length> -DLATENT_RANK=<value length>"
#endif

constexpr int ROW = LATENT_ROW, RANK = LATENT_RANK;
static_assert(ROW % 8 == 0 && RANK % 32 == 0 && RANK >= 32 && RANK <= 512 && RANK <= ROW && ROW <= 832, "row and value sizes");
constexpr int KT = (ROW + 15) / 16;            // k-steps of q.k (a row that ends in half a step is padded with zeros)
constexpr int CPR = ROW / 8;                   // 16-byte chunks of a row that carry data
constexpr int CPR_PAD = KT * 2;                // chunks that the k-steps read
constexpr int ROWP = (ROW + 63) / 64 * 64;     // row length in shared memory: whole 128-byte groups
constexpr int ROWB = ROWP * 2;
constexpr int BM = 64, BN = 32, WARPS = 8, THREADS = WARPS * 32, STAGES = 2;
constexpr int NT = BN / 8;                     // 8-wide column tiles of the scores
constexpr int NTO = RANK / 16;                 // 8-wide column tiles of a warp's half of the output
constexpr int TILE_BYTES = BN * ROWB;
constexpr int SMEM = 128 + BM * ROWB + STAGES * TILE_BYTES;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * ROWB + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Keys tile_start .. tile_start + BN - 1 of the request into a stage; keys outside [key_lo, key_hi) are zeros.
__device__ __forceinline__ void load_keys(uint32_t dst, const bf16* __restrict__ pages, const int* __restrict__ table,
                                          int tile_start, int key_lo, int key_hi, int page_size, int page_shift) {
    for (int idx = threadIdx.x; idx < BN * CPR_PAD; idx += THREADS) {
        const int row = idx / CPR_PAD, chunk = idx % CPR_PAD;
        const int key = tile_start + row;
        const bool valid = key >= key_lo && key < key_hi && chunk < CPR;
        const bf16* src = pages;
        if (valid) src = pages + ((size_t)table[key >> page_shift] * page_size + (key & (page_size - 1))) * ROW + chunk * 8;
        cp_async16(dst + swz(row, chunk), src, valid);
    }
}

__global__ void __launch_bounds__(THREADS, 1)
latent_mma_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                  const bf16* __restrict__ pages, const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                  const int* __restrict__ req_ctx_len, const int* __restrict__ block_table, int max_pages, int heads,
                  int page_size, int window, float scale2, int skip_single, int q_rows, int split_tiles, int max_splits,
                  float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ unsigned char smem_raw[];
    pdl_begin();
    const int r = blockIdx.y;
    const int q_len = req_q_len[r];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int rows = q_len * heads;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;        // the tiles with the most keys start first
    const int row0 = tile * q_rows;                                // q_rows: 64, or 16 in a launch whose requests have no more
    if (row0 >= rows) return;
    const int ctx = req_ctx_len[r], q_start = req_q_start[r], pos0 = ctx - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp >> 1, half = warp & 1;                  // 16 rows; which half of the value's columns
    const uint32_t base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 127u) & ~127u;
    const uint32_t q_s = base + STAGES * TILE_BYTES;
    const int* table = block_table + (size_t)r * max_pages;
    const int page_shift = 31 - __clz(page_size);

    // the keys that the CTA's rows see: from the first row's first key to the last row's position
    const int last_row = min(rows, row0 + q_rows) - 1;
    const int pos_lo = pos0 + row0 / heads, pos_hi = pos0 + last_row / heads;
    const int key_lo = first_visible_key(pos_lo, window), key_hi = pos_hi + 1;
    int t0 = key_lo / BN, t1 = (key_hi + BN - 1) / BN;
    // a single token's keys may be cut into splits of `split_tiles` tiles, one CTA each (blockIdx.z); the others run whole
    int num_splits = 1;
    if (split_tiles > 0 && q_len == 1) {
        num_splits = (t1 - t0 + split_tiles - 1) / split_tiles;
        if ((int)blockIdx.z >= num_splits) return;
        t0 += (int)blockIdx.z * split_tiles;
        t1 = min(t1, t0 + split_tiles);
    } else if (blockIdx.z > 0) {
        return;
    }

    int pos_r[2], first_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = row0 + group * 16 + (lane >> 2) + i * 8;
        pos_r[i] = m < rows ? pos0 + m / heads : -1;               // a row past the end sees no key
        first_r[i] = first_visible_key(pos_r[i], window);
    }
    // the keys that the warp's 16 rows see
    const int warp_first_row = row0 + group * 16;
    const bool warp_has_rows = warp_first_row < rows && group * 16 < q_rows;
    const int warp_pos_lo = pos0 + min(rows - 1, warp_first_row) / heads;
    const int warp_pos_hi = pos0 + min(rows - 1, warp_first_row + 15) / heads;
    const int warp_key_lo = first_visible_key(warp_pos_lo, window);

    // the queries: row m is (token m / heads, head m % heads)
    for (int idx = threadIdx.x; idx < q_rows * CPR_PAD; idx += THREADS) {
        const int row = idx / CPR_PAD, chunk = idx % CPR_PAD;
        const int m = row0 + row;
        const bool valid = m < rows && chunk < CPR;
        const bf16* src = q;
        if (valid) src = q + (size_t)(q_start + m / heads) * q_stride + (size_t)(m % heads) * ROW + chunk * 8;
        cp_async16(q_s + swz(row, chunk), src, valid);
    }
    load_keys(base, pages, table, t0 * BN, key_lo, key_hi, page_size, page_shift);
    cp_commit();

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NTO][4];
#pragma unroll
    for (int n = 0; n < NTO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_chunk = lane >> 4;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_chunk = (lane >> 3) & 1;
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_chunk = lane >> 4;
    const int col_chunk0 = half * (RANK / 16);                     // the warp's first 16-byte chunk of the value's columns

    for (int t = t0; t < t1; ++t) {
        const int s = (t - t0) % STAGES;
        if (t + 1 < t1) {
            load_keys(base + ((t + 1 - t0) % STAGES) * TILE_BYTES, pages, table, (t + 1) * BN, key_lo, key_hi, page_size, page_shift);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const uint32_t k_tile = base + s * TILE_BYTES;
        const int key_base = t * BN;
        if (warp_has_rows && key_base <= warp_pos_hi && key_base + BN > warp_key_lo) {
            float sc[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll 4
            for (int kt = 0; kt < KT; ++kt) {
                uint32_t a[4];
                ldsm4(q_s + swz(group * 16 + a_row, kt * 2 + a_chunk), a);
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t b[4];
                    ldsm4(k_tile + swz(np * 16 + b_row, kt * 2 + b_chunk), b);
                    mma16816(sc[2 * np], a, b[0], b[1]);
                    mma16816(sc[2 * np + 1], a, b[2], b[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = key_base + n * 8 + (lane & 3) * 2 + (c & 1);
                    const int i = c >> 1;
                    const bool ok = key <= pos_r[i] && key >= first_r[i];
                    sc[n][c] = ok ? sc[n][c] * scale2 : -INFINITY;
                    mx[i] = fmaxf(mx[i], sc[n][c]);
                }
            float corr[2], mbase[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m_run[i], mx[i]);
                mbase[i] = m_new == -INFINITY ? 0.f : m_new;       // a row that has seen no key yet
                corr[i] = exp2f(m_run[i] - mbase[i]);              // exp2(-inf) = 0 for the first keys
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
#pragma unroll
            for (int n = 0; n < NTO; ++n) {
                o[n][0] *= corr[0]; o[n][1] *= corr[0];
                o[n][2] *= corr[1]; o[n][3] *= corr[1];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    sc[n][c] = exp2f(sc[n][c] - mbase[c >> 1]);
                    l_run[c >> 1] += sc[n][c];
                }
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                uint32_t p[4];
                p[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                p[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                p[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                p[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int np = 0; np < NTO / 2; ++np) {
                    uint32_t b[4];
                    ldsm4t(k_tile + swz(kk * 16 + v_row, col_chunk0 + np * 2 + v_chunk), b);
                    mma16816(o[2 * np], p, b[0], b[1]);
                    mma16816(o[2 * np + 1], p, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                           // the stage is free for the tile after next
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    if (num_splits > 1) {                 // this split's maximum, sum and unnormalised output; merged in split order afterwards
        if (!warp_has_rows) return;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int m = group * 16 + (lane >> 2) + i * 8;             // row0 is 0: a single token's rows are its heads
            if (m >= rows) continue;
            const size_t at = ((size_t)r * max_splits + blockIdx.z) * heads + m;
            if (half == 0 && (lane & 3) == 0) { part_ml[at * 2] = m_run[i]; part_ml[at * 2 + 1] = l_run[i]; }
            float* dst = part_o + at * RANK + half * (RANK / 2) + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < NTO; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = row0 + group * 16 + (lane >> 2) + i * 8;
        if (m >= rows || !warp_has_rows) continue;
        const float inv = 1.0f / l_run[i];
        bf16* dst = out + (size_t)(q_start + m / heads) * out_stride + (size_t)(m % heads) * RANK + half * (RANK / 2) + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NTO; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
}

// The splits of a single token's keys into one output row per head, in split order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(bf16* __restrict__ out, int out_stride, const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                    const int* __restrict__ req_ctx_len, int heads, int window, int split_tiles, int max_splits,
                    const float* __restrict__ part_o, const float* __restrict__ part_ml) {
    pdl_begin();
    const int h = blockIdx.x, r = blockIdx.y;
    if (req_q_len[r] != 1) return;
    const int pos = req_ctx_len[r] - 1;
    const int t0 = first_visible_key(pos, window) / BN, t1 = (pos + BN) / BN;
    const int num_splits = (t1 - t0 + split_tiles - 1) / split_tiles;
    if (num_splits <= 1) return;
    const size_t at0 = (size_t)r * max_splits * heads + h;
    float top = -INFINITY;
    for (int z = 0; z < num_splits; ++z) top = fmaxf(top, part_ml[(at0 + (size_t)z * heads) * 2]);
    float sum = 0.f;
    for (int z = 0; z < num_splits; ++z) {
        const size_t at = at0 + (size_t)z * heads;
        sum += part_ml[at * 2 + 1] * exp2f(part_ml[at * 2] - top);
    }
    const float inv = 1.0f / sum;
    bf16* dst = out + (size_t)req_q_start[r] * out_stride + (size_t)h * RANK;
    for (int c = threadIdx.x; c < RANK; c += 128) {
        float acc = 0.f;
        for (int z = 0; z < num_splits; ++z) {
            const size_t at = at0 + (size_t)z * heads;
            acc += part_o[at * RANK + c] * exp2f(part_ml[at * 2] - top);
        }
        dst[c] = __float2bfloat16_rn(acc * inv);
    }
}

WLLM_API int wllm_latent_attention_mma_row() { return ROW; }
WLLM_API int wllm_latent_attention_mma_rank() { return RANK; }

// q: [n, heads * ROW] (row stride q_stride), out: [n, heads * RANK]; pages: [pool pages][page_size][ROW];
// requests by start, length and context; `max_q_len` the most tokens any request brings.
WLLM_API int wllm_latent_attention_mma(const void* q, int q_stride, void* out, int out_stride, const void* pages,
                                       const int* req_q_start, const int* req_q_len, const int* req_ctx_len,
                                       const int* block_table, int max_pages, int requests, int max_q_len, int heads,
                                       int page_size, int window, float scale, int skip_single, int split_tiles, int max_splits,
                                       float* scratch, cudaStream_t stream) {
    if (requests <= 0 || max_q_len <= 0) return WLLM_OK;
    if (split_tiles < 0 || (split_tiles > 0 && (max_splits < 1 || max_splits > 65535 || scratch == nullptr || heads > BM)))
        return WLLM_BAD_SIZE;
    if (heads <= 0 || page_size <= 0 || (page_size & (page_size - 1)) || max_pages <= 0 || requests > 65535) return WLLM_BAD_SIZE;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3) || ((uintptr_t)pages & 15))
        return WLLM_BAD_ALIGN;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(latent_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    // a launch whose requests have at most 16 rows each keeps 16 query rows in shared memory: two CTAs fit an SM
    const int q_rows = (long long)max_q_len * heads <= 16 ? 16 : BM;
    const long long tiles = ((long long)max_q_len * heads + q_rows - 1) / q_rows;
    if (tiles > 0x7fffffffLL) return WLLM_BAD_SIZE;
    if (split_tiles == 0) max_splits = 1;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)requests * max_splits * heads * RANK : nullptr;
    const int smem = 128 + q_rows * ROWB + STAGES * TILE_BYTES;
    const int st = wllm_launch(latent_mma_kernel, dim3((unsigned)tiles, requests, max_splits), THREADS, smem, stream, (const bf16*)q,
                               q_stride, (bf16*)out, out_stride, (const bf16*)pages, req_q_start, req_q_len, req_ctx_len, block_table,
                               max_pages, heads, page_size, window, scale * LOG2E, skip_single, q_rows, split_tiles, max_splits,
                               part_o, part_ml);
    if (st || max_splits == 1) return st;
    return wllm_launch(latent_merge_kernel, dim3(heads, requests), 128, 0, stream, (bf16*)out, out_stride, req_q_start, req_q_len,
                       req_ctx_len, heads, window, split_tiles, max_splits, (const float*)part_o, (const float*)part_ml);
}

// Floats of scratch for `requests` single tokens whose keys are cut into up to `max_splits` splits.
WLLM_API long long wllm_latent_attention_mma_scratch_floats(int requests, int heads, int max_splits) {
    return (long long)requests * max_splits * heads * (RANK + 2);
}
