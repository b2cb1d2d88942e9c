// Routed experts: every token runs `top` of E small gated feed-forward units, chosen by a router.
//
//   route    z = W_router h in 32-bit (W_router is held in 32-bit; h as the norm left it), s = softmax(z) over all
//            experts.  The experts form `groups` equal groups of neighbours; a group's score is its best expert's, and
//            only experts of the `groups_kept` best groups can be chosen.  The `top` best of those are the token's
//            experts, in descending order of score (ties: the lower index first), weighted by their scores as they
//            are.  A shared unit's gate, sigmoid(w_gate . h), is worked out along the way.  One CTA a token; every
//            dot product is a lane's strided chain and the warp's tree, so a token's choice and weights do not depend
//            on the batch.
//   plan     the (token, rank) pairs sorted by expert, stably: count[e], offset[e], sorted[r] = pair, place[pair] = r.
//            A warp an expert, by ballots over the pair list; no atomics, so the order is the same every time.
//   experts  grouped products over the sorted rows: act = unit(gate_e a, up_e a) for the rows of expert e (a gathered
//            from the tokens' rows), then y = down_e act, 32-bit accumulation, each output one ascending chain over k.
//            A CTA takes a tile of rows of ONE expert and a tile of columns; the grid is sized from the pair count
//            and E alone (tiles that find no rows leave at once), so a captured step can replay it.
//            Steps of many rows run these products on the tensor-memory kernel instead (gemm_bf16_tc.cu, grouped), over the
//            tokens' rows copied into sorted order (moe_gather) and the table of row tiles that the plan writes.
//   combine  out[token] = sum over the token's ranks, in rank order, of weight * y[place] (+ gate * shared unit).
//
// Two more forms.  Scores: softmax over all experts, or (score_mode 1) sigmoid(z) expert by expert, not normalised (without
// groups the experts are then chosen by z itself: the same order, and no ties where large logits all round to a score of 1).  Unit
// (MODE 2): an expert without a gate, down(relu(up (s a))^2), whose input is multiplied by the pair's score s: the up product
// is linear, so s multiplies its 32-bit sums in front of the activation; the combine then adds the experts' outputs as they are.
//
// The gated unit is the clamped one: g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(slope g) (u + 1).
#include "common.cuh"

constexpr int MOE_MAX_EXPERTS = 1024;

// A CTA takes `tpb` tokens: a warp an expert (and one for the shared gate) reads its row of the router once and runs it
// against the CTA's tokens; then a warp a token does the softmax and the choice.
template <typename T>
__global__ void __launch_bounds__(1024)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ w_router, const float* __restrict__ w_gate,
                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ gate_out, int n, int H, int E, int top,
                 int groups, int groups_kept, int tpb, int score_mode) {
    extern __shared__ float route_smem[];          // [tpb][H] the tokens' rows, [tpb][E] scores, [tpb][groups] group scores
    float* hs_all = route_smem;
    float* sc_all = hs_all + (size_t)tpb * H;
    float* gs_all = sc_all + (size_t)tpb * E;
    pdl_begin();
    const int t0 = blockIdx.x * tpb, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int here = min(tpb, n - t0);
    for (int i = threadIdx.x; i < here * H; i += blockDim.x) hs_all[i] = to_f32(h[(size_t)t0 * H + i]);
    __syncthreads();
    constexpr int TB = 4;                          // tokens a pass over the router's row
    for (int e = warp; e < E + (w_gate != nullptr ? 1 : 0); e += nwarps) {
        const float* w = e < E ? w_router + (size_t)e * H : w_gate;
        for (int j0 = 0; j0 < here; j0 += TB) {
            // a lane's share of a row as four chains (elements c .. c+3 of every 128), added in a fixed order: the sum
            // depends on the token's row and H alone, not on the tokens beside it
            float a4[TB][4];
#pragma unroll
            for (int j = 0; j < TB; ++j) a4[j][0] = a4[j][1] = a4[j][2] = a4[j][3] = 0.f;
            if ((H & 3) == 0) {
                const float* hrow[TB];
#pragma unroll
                for (int j = 0; j < TB; ++j) hrow[j] = hs_all + (size_t)min(j0 + j, here - 1) * H;
#pragma unroll 4
                for (int c = lane * 4; c < H; c += 128) {           // several of the router's 16-byte loads in flight
                    const float4 wv = *reinterpret_cast<const float4*>(w + c);
#pragma unroll
                    for (int j = 0; j < TB; ++j) {
                        const float4 hv = *reinterpret_cast<const float4*>(hrow[j] + c);
                        a4[j][0] = fmaf(wv.x, hv.x, a4[j][0]); a4[j][1] = fmaf(wv.y, hv.y, a4[j][1]);
                        a4[j][2] = fmaf(wv.z, hv.z, a4[j][2]); a4[j][3] = fmaf(wv.w, hv.w, a4[j][3]);
                    }
                }
            } else {
                for (int c = lane; c < H; c += 32)
#pragma unroll
                    for (int j = 0; j < TB; ++j) a4[j][0] = fmaf(w[c], hs_all[(size_t)min(j0 + j, here - 1) * H + c], a4[j][0]);
            }
#pragma unroll
            for (int j = 0; j < TB; ++j) {
                const float acc = warp_sum((a4[j][0] + a4[j][1]) + (a4[j][2] + a4[j][3]));
                if (lane == 0 && j0 + j < here) {
                    if (e < E) sc_all[(size_t)(j0 + j) * E + e] = acc; else gate_out[t0 + j0 + j] = 1.0f / (1.0f + expf(-acc));
                }
            }
        }
    }
    __syncthreads();
    for (int j = warp; j < here; j += nwarps) {
        const int t = t0 + j;
        float* sc = sc_all + (size_t)j * E;
        float* gs = gs_all + (size_t)j * groups;
        if (score_mode == 1 && groups == 1) {
            // sigmoid scores without groups: the choice is made on the logits themselves (the sigmoid keeps their order, but
            // large logits all round to a score of 1 and would tie); the weights are the chosen logits' sigmoids
            for (int k = 0; k < top; ++k) {
                float best = -INFINITY; int at = 0x7fffffff;
                for (int e = lane; e < E; e += 32) { const float v = sc[e]; if (v > best || (v == best && e < at)) { best = v; at = e; } }
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
                }
                if (lane == 0) {
                    chosen[(size_t)t * top + k] = at;
                    weights[(size_t)t * top + k] = 1.0f / (1.0f + expf(-best));
                    sc[at] = -INFINITY;
                }
                __syncwarp();
            }
            continue;
        }
        if (score_mode == 1) {
            for (int e = lane; e < E; e += 32) sc[e] = 1.0f / (1.0f + expf(-sc[e]));
        } else {
            float m = -INFINITY;
            for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
            m = warp_max(m);
            float sum = 0.f;
            for (int e = lane; e < E; e += 32) { const float p = expf(sc[e] - m); sc[e] = p; sum += p; }
            sum = warp_sum(sum);
            const float inv = 1.0f / sum;
            for (int e = lane; e < E; e += 32) sc[e] *= inv;
        }
        __syncwarp();
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int i = 0; i < per; ++i) best = fmaxf(best, sc[g * per + i]);
            gs[g] = best;
        }
        __syncwarp();
        // the groups that stay: groups_kept times the best one left (ties: the lower index); the others' experts leave
        if (groups_kept < groups) {
            for (int pick = 0; pick < groups_kept; ++pick) {
                float best = -INFINITY; int at = 0x7fffffff;
                for (int g = lane; g < groups; g += 32) { const float v = gs[g]; if (v > best) { best = v; at = g; } }
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
                }
                if (lane == 0) gs[at] = -2.0f;              // marked as kept (scores lie in [0, 1])
                __syncwarp();
            }
            for (int e = lane; e < E; e += 32) if (gs[e / per] != -2.0f) sc[e] = -1.0f;
            __syncwarp();
        }
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY; int at = 0x7fffffff;
            for (int e = lane; e < E; e += 32) { const float v = sc[e]; if (v > best) { best = v; at = e; } }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0) { chosen[(size_t)t * top + k] = at; weights[(size_t)t * top + k] = best; sc[at] = -3.0f; }
            __syncwarp();
        }
    }
}

// The pair list is cut into `segs` segments of seg_len pairs (a multiple of 128) so that long lists are scanned by segs
// warps an expert.  grid: E * segs warps (4 a CTA).  partial[seg * E + e] = pairs of the segment whose expert is e.
__global__ void __launch_bounds__(128) moe_count_kernel(const int* __restrict__ chosen, int pairs, int E, int segs, int seg_len,
                                                        int* __restrict__ partial) {
    pdl_begin();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= E * segs) return;
    const int e = w % E, seg = w / E;
    const int lo = seg * seg_len, hi = min(pairs, lo + seg_len);
    int c = 0;
    for (int p0 = lo; p0 < hi; p0 += 128) {          // four loads in flight a lane
        bool mine[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { const int p = p0 + 32 * u + lane; mine[u] = p < hi && chosen[p] == e; }
#pragma unroll
        for (int u = 0; u < 4; ++u) c += __popc(__ballot_sync(0xffffffffu, mine[u]));
    }
    if (lane == 0) partial[seg * E + e] = c;
}

// count[e] = pairs of expert e, offset[e] = count[0] + .. + count[e-1] (offset[E] = pairs); the pairs of expert e in ascending
// order fill the sorted rows from offset[e]: sorted[r] = pair, place[pair] = r.  The warp of (expert, segment) places its
// segment's pairs behind those of the segments before it.
// With `tiles` (null: none): the table of row tiles of `tile_rows` rows of one expert each, for the products that walk it:
// tiles[0] = their number, then (expert, first sorted row, rows) a tile, expert by expert.
__global__ void __launch_bounds__(128) moe_place_kernel(const int* __restrict__ chosen, int pairs, int E, int segs, int seg_len,
                                                        const int* __restrict__ partial, int* __restrict__ count,
                                                        int* __restrict__ offset, int* __restrict__ sorted, int* __restrict__ place,
                                                        int* __restrict__ tiles, int tile_rows) {
    pdl_begin();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= E * segs) return;
    const int e = w % E, seg = w / E;
    int before = 0, tiles_before = 0;
    for (int j = lane; j < e; j += 32) {
        int c = 0;
        for (int s2 = 0; s2 < segs; ++s2) c += partial[s2 * E + j];
        before += c;
        if (tiles) tiles_before += (c + tile_rows - 1) / tile_rows;
    }
    for (int o = 16; o > 0; o >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, o);
        tiles_before += __shfl_xor_sync(0xffffffffu, tiles_before, o);
    }
    int mine_total = 0, mine_before = 0;
    for (int s2 = 0; s2 < segs; ++s2) {
        const int c = partial[s2 * E + e];
        mine_total += c;
        if (s2 < seg) mine_before += c;
    }
    if (seg == 0) {
        if (lane == 0) {
            count[e] = mine_total;
            offset[e] = before;
            if (e == E - 1) offset[E] = before + mine_total;
        }
        if (tiles) {
            const int n_tiles = (mine_total + tile_rows - 1) / tile_rows;
            for (int t = lane; t < n_tiles; t += 32) {
                int* entry = tiles + 1 + 3 * (tiles_before + t);
                entry[0] = e; entry[1] = before + t * tile_rows; entry[2] = min(tile_rows, mine_total - t * tile_rows);
            }
            if (e == E - 1 && lane == 0) tiles[0] = tiles_before + n_tiles;
        }
    }
    int at = before + mine_before;
    const int lo = seg * seg_len, hi = min(pairs, lo + seg_len);
    for (int p0 = lo; p0 < hi; p0 += 128) {          // four loads in flight a lane; the pairs still go in ascending order
        bool mine[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { const int p = p0 + 32 * u + lane; mine[u] = p < hi && chosen[p] == e; }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const unsigned b = __ballot_sync(0xffffffffu, mine[u]);
            if (mine[u]) {
                const int r = at + __popc(b & ((1u << lane) - 1u));
                sorted[r] = p0 + 32 * u + lane;
                place[p0 + 32 * u + lane] = r;
            }
            at += __popc(b);
        }
    }
}

constexpr int GM = 32, GN = 64, GK = 16;

// One tile of rows (of one expert) by one tile of columns.  GATED: w holds [E][2 N][K] (gate rows, then up rows), the
// rows of a are gathered (token = sorted[r] / top) and out[r][c] = unit(gate, up) in TO; else w is [E][N][K], the rows
// of a are the sorted rows and out is 32-bit.  Thread (ty, tx) of 16 x 16 owns rows ty, ty + 16 and columns tx + 16 j.
// MODE 2: w is [E][N][K], the rows of a are gathered as for the gated unit, and out[r][c] = relu(row_w[sorted[r]] * sum)^2 in TO.
template <typename T, typename TO, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w, TO* __restrict__ out, int N, int K,
                   const int* __restrict__ offset, const int* __restrict__ sorted, int E, int top, float limit, float slope,
                   const float* __restrict__ row_w) {
    constexpr bool GATED = MODE == 1, GATHER = MODE != 0;
    __shared__ float As[GK][GM + 1];
    __shared__ float Ws[GATED ? 2 : 1][GK][GN + 1];
    __shared__ int s_expert, s_row0, s_rows;
    pdl_begin();
    if (threadIdx.x == 0) {
        // the tile's expert: tiles are dealt expert by expert, ceil(count / GM) each
        int tile = blockIdx.y, e = 0, found = -1, row0 = 0, rows = 0;
        for (; e < E; ++e) {
            const int lo = offset[e], cnt = offset[e + 1] - lo, tiles = (cnt + GM - 1) / GM;
            if (tile < tiles) { found = e; row0 = lo + tile * GM; rows = min(GM, cnt - tile * GM); break; }
            tile -= tiles;
        }
        s_expert = found; s_row0 = row0; s_rows = rows;
    }
    __syncthreads();
    const int e = s_expert;
    if (e < 0) return;
    const int row0 = s_row0, rows = s_rows, col0 = blockIdx.x * GN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    float acc[GATED ? 2 : 1][2][4];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;
    // which row of `a` each of the tile's rows reads
    const int lr = threadIdx.x >> 3;                 // 0..31: the row this thread loads (two k each)
    int src_row = -1;
    if (lr < rows) src_row = GATHER ? sorted[row0 + lr] / top : row0 + lr;
    for (int k0 = 0; k0 < K; k0 += GK) {
        {
            const int kk = (threadIdx.x & 7) * 2;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int k = k0 + kk + u;
                As[kk + u][lr] = (src_row >= 0 && k < K) ? to_f32(a[(size_t)src_row * a_stride + k]) : 0.f;
            }
        }
#pragma unroll
        for (int g = 0; g < (GATED ? 2 : 1); ++g) {
            for (int idx = threadIdx.x; idx < GN * GK; idx += 256) {
                const int c = idx / GK, kk = idx % GK, col = col0 + c, k = k0 + kk;
                Ws[g][kk][c] = (col < N && k < K) ? to_f32(we[((size_t)g * N + col) * K + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            const float a0 = As[kk][ty], a1 = As[kk][ty + 16];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float wv = Ws[g][kk][tx + 16 * j];
                    acc[g][0][j] = fmaf(a0, wv, acc[g][0][j]);
                    acc[g][1][j] = fmaf(a1, wv, acc[g][1][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty + 16 * i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col0 + tx + 16 * j;
            if (col >= N) continue;
            float v = acc[0][i][j];
            if (GATED) {
                const float g = fminf(v, limit), u = fminf(fmaxf(acc[GATED ? 1 : 0][i][j], -limit), limit);
                v = (g / (1.0f + expf(-slope * g))) * (u + 1.0f);
            }
            if (MODE == 2) {
                v = fmaxf(row_w ? v * row_w[sorted[row0 + r]] : v, 0.f);
                v *= v;
            }
            out[(size_t)(row0 + r) * N + col] = from_f32<TO>(v);
        }
    }
}

// The same products for bfloat16 operands on the tensor cores (mma.sync m16n8k16, 32-bit accumulators): a CTA of eight
// warps takes 64 rows of one expert by 128 rows of W (128 output columns, or, gated, 64 gate rows and the 64 up rows of
// the same columns, laid out so that a thread holds gate and up of the same output element), K in blocks of 32 through
// a ring of three cp.async stages; rows of A are gathered through `sorted` while they are copied.  K in steps of 8.
constexpr int TM = 64, TN = 128, TK = 32, TPITCH = TK + 8, TSTAGES = 3;      // a pitch of 80 bytes: ldmatrix without bank conflicts
// (blocks of 64 of K were measured too: 83 KB a CTA leave two CTAs an SM instead of four, 334 -> 362 us at 8,192 rows)
constexpr int T_SMEM = TSTAGES * (TM + TN) * TPITCH * 2;

__device__ __forceinline__ void moe_cp16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void moe_ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void moe_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The tile's expert and rows from the offsets, by one warp: tiles are dealt expert by expert, ceil(count / rows_per_tile) each.
__device__ __forceinline__ void moe_find_tile(const int* __restrict__ offset, int E, int rows_per_tile, int tile, int lane,
                                              int& expert, int& row0, int& rows) {
    expert = -1; row0 = 0; rows = 0;
    int base = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int lo = e < E ? offset[e] : 0, cnt = e < E ? offset[e + 1] - lo : 0;
        const int tiles = (cnt + rows_per_tile - 1) / rows_per_tile;
        int incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
        const int first = base + incl - tiles;
        const bool mine = tile >= first && tile < base + incl;
        const unsigned b = __ballot_sync(0xffffffffu, mine);
        if (b) {
            const int src = __ffs(b) - 1;
            const int k = tile - __shfl_sync(0xffffffffu, first, src);
            expert = e0 + src;
            row0 = __shfl_sync(0xffffffffu, lo, src) + k * rows_per_tile;
            rows = min(rows_per_tile, __shfl_sync(0xffffffffu, cnt, src) - k * rows_per_tile);
            return;
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
}

template <typename TO, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_mma_kernel(const bf16* __restrict__ a, int a_stride, const bf16* __restrict__ w, TO* __restrict__ out, int N, int K,
                       const int* __restrict__ offset, const int* __restrict__ sorted, int E, int top, float limit, float slope,
                       const float* __restrict__ row_w) {
    constexpr bool GATED = MODE == 1, GATHER = MODE != 0;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    bf16 (*As)[TM][TPITCH] = reinterpret_cast<bf16 (*)[TM][TPITCH]>(moe_smem);
    bf16 (*Ws)[TN][TPITCH] = reinterpret_cast<bf16 (*)[TN][TPITCH]>(moe_smem + TSTAGES * TM * TPITCH * 2);
    __shared__ int s_tile[3];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        int e, r0, rs;
        moe_find_tile(offset, E, TM, blockIdx.y, lane, e, r0, rs);
        if (lane == 0) { s_tile[0] = e; s_tile[1] = r0; s_tile[2] = rs; }
    }
    __syncthreads();
    const int e = s_tile[0];
    if (e < 0) return;
    const int row0 = s_tile[1], rows = s_tile[2];
    constexpr int COLS = GATED ? TN / 2 : TN;               // output columns of a tile
    const int col0 = blockIdx.x * COLS;
    const bf16* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    // what this thread copies a stage: TK / 32 16-byte pieces of a row of A (64 rows) and of two rows of W (128 rows)
    const int a_row = threadIdx.x >> 2, piece0 = threadIdx.x & 3;
    const bf16* a_src = nullptr;
    if (a_row < rows) a_src = a + (size_t)(GATHER ? sorted[row0 + a_row] / top : row0 + a_row) * a_stride;
    const bf16* w_src[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = a_row + 64 * u;                       // row of the W tile
        int col;
        if (GATED) { const int wn = r >> 5, rr = r & 31; col = ((rr >> 4) ? N : 0) + col0 + 16 * wn + (rr & 15); if (col0 + 16 * wn + (rr & 15) >= N) col = -1; }
        else { col = col0 + r; if (col >= N) col = -1; }
        w_src[u] = col >= 0 ? we + (size_t)col * K : nullptr;
    }
    auto load = [&](int kb, int stage) {
#pragma unroll
        for (int pc = 0; pc < TK / 32; ++pc) {
            const int piece = piece0 + 4 * pc, k = kb * TK + piece * 8;
            const bool in_k = k < K;
            moe_cp16((uint32_t)__cvta_generic_to_shared(&As[stage][a_row][piece * 8]), a_src ? a_src + k : a, a_src != nullptr && in_k);
#pragma unroll
            for (int u = 0; u < 2; ++u)
                moe_cp16((uint32_t)__cvta_generic_to_shared(&Ws[stage][a_row + 64 * u][piece * 8]), w_src[u] ? w_src[u] + k : w,
                         w_src[u] != nullptr && in_k);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int wm = warp & 1, wn = warp >> 1;                // 2 x 4 warps: 32 rows by 32 rows of W each
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    const int kblocks = (K + TK - 1) / TK;
    for (int s0 = 0; s0 < TSTAGES - 1; ++s0) {
        if (s0 < kblocks) load(s0, s0); else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kb = 0; kb < kblocks; ++kb) {
        asm volatile("cp.async.wait_group %0;" ::"n"(TSTAGES - 2) : "memory");
        __syncthreads();                                    // block kb is here for everyone; the stage of block kb-1 is free
        if (kb + TSTAGES - 1 < kblocks) load(kb + TSTAGES - 1, (kb + TSTAGES - 1) % TSTAGES);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = kb % TSTAGES;
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk) {
            uint32_t af[2][4], bfr[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
                moe_ldsm4((uint32_t)__cvta_generic_to_shared(&As[st][wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk * 16 + (lane >> 4) * 8]), af[mi]);
#pragma unroll
            for (int nj = 0; nj < 2; ++nj)
                moe_ldsm4((uint32_t)__cvta_generic_to_shared(&Ws[st][wn * 32 + nj * 16 + (lane & 7) + (lane >> 4) * 8][kk * 16 + ((lane >> 3) & 1) * 8]), bfr[nj]);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int nj = 0; nj < 2; ++nj) {
                    moe_mma(acc[mi][2 * nj], af[mi], bfr[nj][0], bfr[nj][1]);
                    moe_mma(acc[mi][2 * nj + 1], af[mi], bfr[nj][2], bfr[nj][3]);
                }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 32 + mi * 16 + (lane >> 2) + half * 8;
            if (r >= rows) continue;
            TO* orow = out + (size_t)(row0 + r) * N;
            const float rw = (MODE == 2 && row_w) ? row_w[sorted[row0 + r]] : 1.0f;
#pragma unroll
            for (int ni = 0; ni < (GATED ? 2 : 4); ++ni)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int col = GATED ? col0 + 16 * wn + 8 * ni + (lane & 3) * 2 + c : col0 + wn * 32 + ni * 8 + (lane & 3) * 2 + c;
                    if (col >= N) continue;
                    float v = acc[mi][ni][half * 2 + c];
                    if (GATED) {
                        const float g = fminf(v, limit), u = fminf(fmaxf(acc[mi][ni + 2][half * 2 + c], -limit), limit);
                        v = (g / (1.0f + expf(-slope * g))) * (u + 1.0f);
                    }
                    if (MODE == 2) { v = fmaxf(v * rw, 0.f); v *= v; }
                    orow[col] = from_f32<TO>(v);
                }
        }
}

// out[t][c] = sum_k weights[t][k] * y[place[t top + k]][c]  (+ gate[t] * shared[t][c], shared a tensor of TS or `parts`
// 32-bit partial sums added in order first)
// Many rows: a CTA of a few warps a token, one load after the other a thread (other CTAs hide the wait).
template <typename TS>
__global__ void __launch_bounds__(256)
moe_combine_rows_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights, int top,
                        const TS* __restrict__ shared, int parts, size_t part_stride, const float* __restrict__ gate,
                        float* __restrict__ out, int H) {
    pdl_begin();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) {
            // every product and sum rounded on its own, in both kernels: one result whichever serves the row
            const float term = __fmul_rn(weights ? weights[(size_t)t * top + k] : 1.0f, y[(size_t)place[(size_t)t * top + k] * H + c]);
            v = k == 0 ? term : __fadd_rn(v, term);
        }
        if (shared != nullptr) {
            float s = 0.f;
            for (int p = 0; p < parts; ++p) {
                const float part = to_f32(shared[(size_t)p * part_stride + (size_t)t * H + c]);
                s = p == 0 ? part : __fadd_rn(s, part);
            }
            v = fmaf(gate[t], s, v);
        }
        out[(size_t)t * H + c] = v;
    }
}

// Few rows (a decode step): a thread a column or two, the experts' rows and the shared unit's partial sums all in flight.  The
// arithmetic of an output element is that of the kernel above.
template <typename TS>
__global__ void __launch_bounds__(1024)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights, int top,
                   const TS* __restrict__ shared, int parts, size_t part_stride, const float* __restrict__ gate,
                   float* __restrict__ out, int H) {
    __shared__ int s_place[64];
    __shared__ float s_weight[64];
    pdl_begin();
    const int t = blockIdx.x;
    for (int k = threadIdx.x; k < min(top, 64); k += blockDim.x) { s_place[k] = place[(size_t)t * top + k]; s_weight[k] = weights ? weights[(size_t)t * top + k] : 1.0f; }
    __syncthreads();
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = 0.f;
        for (int k0 = 0; k0 < top; k0 += 8) {          // eight of the experts' rows in flight; the sum is in rank order
            float term[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = k0 + u;
                term[u] = 0.f;
                if (k < top) {
                    const int row = k < 64 ? s_place[k] : place[(size_t)t * top + k];
                    const float wk = k < 64 ? s_weight[k] : (weights ? weights[(size_t)t * top + k] : 1.0f);
                    term[u] = __fmul_rn(wk, y[(size_t)row * H + c]);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (k0 + u < top) v = (k0 + u == 0) ? term[u] : __fadd_rn(v, term[u]);
        }
        if (shared != nullptr) {
            float s = 0.f;
            for (int p0 = 0; p0 < parts; p0 += 16) {
                float part[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) part[u] = p0 + u < parts ? to_f32(shared[(size_t)(p0 + u) * part_stride + (size_t)t * H + c]) : 0.f;
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (p0 + u < parts) s = (p0 + u == 0) ? part[u] : __fadd_rn(s, part[u]);
            }
            v = fmaf(gate[t], s, v);
        }
        out[(size_t)t * H + c] = v;
    }
}

WLLM_API int wllm_moe_route(const void* h, int dtype, const float* w_router, const float* w_gate, int* chosen, float* weights,
                            float* gate_out, int n, int H, int E, int top, int groups, int groups_kept, int score_mode,
                            cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (score_mode != 0 && score_mode != 1) return WLLM_BAD_SIZE;
    if (H <= 0 || E <= 0 || E > MOE_MAX_EXPERTS || top < 1 || groups < 1 || E % groups != 0 || groups_kept < 1 ||
        groups_kept > groups || top > groups_kept * (E / groups) || (w_gate != nullptr && gate_out == nullptr))
        return WLLM_BAD_SIZE;
    // tokens a CTA: eight once the tokens alone fill the device (each row of the router is then read once for eight), as
    // long as their rows fit in shared memory
    int tpb = n >= 1024 ? 8 : (n >= 296 ? 2 : 1);
    while (tpb > 1 && (size_t)tpb * (H + E + groups) * sizeof(float) > 160 * 1024) tpb >>= 1;
    const size_t smem = (size_t)tpb * (H + E + groups) * sizeof(float);
    if (smem > 200 * 1024) return WLLM_BAD_SIZE;
    const int threads = 32 * (E + 1 < 4 ? 4 : (E + 1 > 32 ? 32 : E + 1));      // a warp an expert (and the shared gate), up to 32
#define GO(T) do { \
        if (smem > 48 * 1024) { \
            const cudaError_t er = cudaFuncSetAttribute(moe_route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (er != cudaSuccess) return 1000 + (int)er; \
        } \
        return wllm_launch(moe_route_kernel<T>, (n + tpb - 1) / tpb, threads, smem, stream, (const T*)h, w_router, w_gate, chosen, weights, \
                           gate_out, n, H, E, top, groups, groups_kept, tpb, score_mode); \
    } while (0)
    if (dtype == WLLM_BF16) GO(bf16);
    if (dtype == WLLM_F32) GO(float);
#undef GO
    return WLLM_BAD_DTYPE;
}

// count [E], offset [E + 1], sorted [pairs], place [pairs]
constexpr int MOE_PLAN_SEGMENTS = 8;

// tiles (null: none): 1 + 3 * (ceil(pairs / tile_rows) + E) ints, the table of row tiles (see moe_place_kernel).
// scratch (null: none): MOE_PLAN_SEGMENTS * E ints; with it, long pair lists are scanned by that many warps an expert.
WLLM_API int wllm_moe_plan_tiles(const int* chosen, int pairs, int E, int* count, int* offset, int* sorted, int* place, int* tiles,
                                 int tile_rows, int* scratch, cudaStream_t stream) {
    if (pairs <= 0) return WLLM_OK;
    if (E <= 0 || E > MOE_MAX_EXPERTS || (tiles != nullptr && tile_rows < 1)) return WLLM_BAD_SIZE;
    const int segs = (scratch != nullptr && pairs >= 2048) ? MOE_PLAN_SEGMENTS : 1;
    const int seg_len = ((pairs + segs - 1) / segs + 127) / 128 * 128;
    int* partial = segs > 1 ? scratch : count;           // one segment: the partial counts are the counts
    const int st = wllm_launch(moe_count_kernel, (E * segs + 3) / 4, 128, 0, stream, chosen, pairs, E, segs, seg_len, partial);
    if (st != WLLM_OK) return st;
    return wllm_launch(moe_place_kernel, (E * segs + 3) / 4, 128, 0, stream, chosen, pairs, E, segs, seg_len, (const int*)partial, count,
                       offset, sorted, place, tiles, tile_rows);
}

WLLM_API int wllm_moe_plan(const int* chosen, int pairs, int E, int* count, int* offset, int* sorted, int* place, cudaStream_t stream) {
    return wllm_moe_plan_tiles(chosen, pairs, E, count, offset, sorted, place, nullptr, 0, nullptr, stream);
}

// out[r] = x[sorted[r] / top]: the tokens' rows in the order of the sorted pairs (K elements of 2 bytes, K in steps of 8)
// row_w (null: none): the row is multiplied by its pair's weight on the way, in 32-bit, rounded once
__global__ void __launch_bounds__(128) moe_gather_kernel(const bf16* __restrict__ x, int x_stride, const int* __restrict__ sorted, int top,
                                                         bf16* __restrict__ out, int K, const float* __restrict__ row_w) {
    pdl_begin();
    const int r = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(sorted[r] / top) * x_stride);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * K);
    if (row_w == nullptr) {
        for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
        return;
    }
    const float s = row_w[sorted[r]];
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
        uint4 v = src[i];
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            h2[e] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        dst[i] = v;
    }
}

WLLM_API int wllm_moe_gather_scaled(const void* x, int x_stride, const int* sorted, int top, void* out, int pairs, int K,
                                    const float* row_w, cudaStream_t stream) {
    if (pairs <= 0) return WLLM_OK;
    if (K <= 0 || K % 8 != 0 || x_stride % 8 != 0 || top < 1) return WLLM_BAD_SIZE;
    if (((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return WLLM_BAD_ALIGN;
    return wllm_launch(moe_gather_kernel, pairs, 128, 0, stream, (const bf16*)x, x_stride, sorted, top, (bf16*)out, K, row_w);
}

WLLM_API int wllm_moe_gather(const void* x, int x_stride, const int* sorted, int top, void* out, int pairs, int K, cudaStream_t stream) {
    return wllm_moe_gather_scaled(x, x_stride, sorted, top, out, pairs, K, nullptr, stream);
}

// unit = 1: a [n][K] rows of tokens (stride a_stride), w [E][2 N][K], out [pairs][N] of the operands' type (the clamped gated unit);
// unit = 0: a [pairs][K] sorted rows, w [E][N][K], out [pairs][N] 32-bit;
// unit = 2: a [n][K] rows of tokens, w [E][N][K], out [pairs][N] of the operands' type = relu(row_w[pair] * (w a))^2 (row_w null: 1).
WLLM_API int wllm_moe_grouped_unit(const void* a, int a_stride, const void* w, void* out, int dtype, int unit, int pairs, int N, int K,
                                   const int* offset, const int* sorted, int E, int top, float limit, float slope, const float* row_w,
                                   cudaStream_t stream) {
    if (pairs <= 0) return WLLM_OK;
    if (N <= 0 || K <= 0 || E <= 0 || E > MOE_MAX_EXPERTS || top < 1 || unit < 0 || unit > 2) return WLLM_BAD_SIZE;
    const dim3 grid((N + GN - 1) / GN, (pairs + GM - 1) / GM + E);
    if (grid.y > 65535) return WLLM_BAD_SIZE;
#define GO(T, TO, M) wllm_launch(moe_grouped_kernel<T, TO, M>, grid, 256, 0, stream, (const T*)a, a_stride, (const T*)w, (TO*)out, N, K, \
                                 offset, sorted, E, top, limit, slope, row_w)
    if (dtype == WLLM_BF16 && K % 8 == 0 && a_stride % 8 == 0 && !((uintptr_t)a & 15) && !((uintptr_t)w & 15)) {
        const int cols = unit == 1 ? TN / 2 : TN;
        const dim3 tgrid((N + cols - 1) / cols, (pairs + TM - 1) / TM + E);
        if (tgrid.y > 65535) return WLLM_BAD_SIZE;
        static bool raised = false;
        if (!raised) {
            cudaError_t er = cudaFuncSetAttribute(moe_grouped_mma_kernel<bf16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM);
            if (er == cudaSuccess) er = cudaFuncSetAttribute(moe_grouped_mma_kernel<float, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM);
            if (er == cudaSuccess) er = cudaFuncSetAttribute(moe_grouped_mma_kernel<bf16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM);
            if (er != cudaSuccess) return 1000 + (int)er;
            raised = true;
        }
#define TGO(TO, M) wllm_launch(moe_grouped_mma_kernel<TO, M>, tgrid, 256, T_SMEM, stream, (const bf16*)a, a_stride, (const bf16*)w, \
                               (TO*)out, N, K, offset, sorted, E, top, limit, slope, row_w)
        return unit == 1 ? TGO(bf16, 1) : unit == 2 ? TGO(bf16, 2) : TGO(float, 0);
#undef TGO
    }
    if (dtype == WLLM_BF16) return unit == 1 ? GO(bf16, bf16, 1) : unit == 2 ? GO(bf16, bf16, 2) : GO(bf16, float, 0);
    if (dtype == WLLM_F32) return unit == 1 ? GO(float, float, 1) : unit == 2 ? GO(float, float, 2) : GO(float, float, 0);
#undef GO
    return WLLM_BAD_DTYPE;
}

WLLM_API int wllm_moe_grouped(const void* a, int a_stride, const void* w, void* out, int dtype, int gated, int pairs, int N, int K,
                              const int* offset, const int* sorted, int E, int top, float limit, float slope, cudaStream_t stream) {
    return wllm_moe_grouped_unit(a, a_stride, w, out, dtype, gated ? 1 : 0, pairs, N, K, offset, sorted, E, top, limit, slope, nullptr, stream);
}

WLLM_API int wllm_moe_combine(const float* y, const int* place, const float* weights, int top, const void* shared, int shared_dtype,
                              int parts, long long part_stride, const float* gate, float* out, int n, int H, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || top < 1 || parts < 1 || (shared != nullptr && gate == nullptr)) return WLLM_BAD_SIZE;
    int threads = H >= 1024 ? 256 : 128;
    if (n <= 64) threads = H >= 2048 ? 1024 : (H >= 1024 ? 512 : threads);      // few rows: a thread a column or two, every load in flight
    const bool few = n <= 64;
    if (shared == nullptr || shared_dtype == WLLM_F32)
        return wllm_launch(few ? moe_combine_kernel<float> : moe_combine_rows_kernel<float>, n, threads, 0, stream, y, place, weights, top,
                           (const float*)shared, parts, (size_t)part_stride, gate, out, H);
    if (shared_dtype == WLLM_BF16 && parts == 1)
        return wllm_launch(few ? moe_combine_kernel<bf16> : moe_combine_rows_kernel<bf16>, n, threads, 0, stream, y, place, weights, top,
                           (const bf16*)shared, parts, (size_t)part_stride, gate, out, H);
    return WLLM_BAD_DTYPE;
}
