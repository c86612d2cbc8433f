// Routed experts: a feed-forward made of many small gated feed-forwards of which every token uses a few.
//
//   route     per token, float32: z = R x (R [experts, width] float32), s = sigmoid(z), choice = s + correction;
//             experts form `groups` equal groups of neighbours, a group's score is the sum of its two largest
//             choices, only experts of the `keep` best groups can be chosen (`top` of them, by choice, ties to
//             the lower index); weights = s of the chosen over their sum (+ 1e-20).  One more row of R, if given,
//             is the gate of a shared expert: sigmoid of its product, one number per token.  The kernel also
//             counts the tokens of every expert (a token's place among its expert's tokens is the count it met).
//   arrange   one block: running sums of the counts (first row of every expert in the order by expert), the
//             list of row tiles for the products, each (token, choice) pair's row in that order and back;
//             the counts are zero again afterwards.
//   products  over the rows in the order by expert, a tile of rows of ONE expert per block, the rows of the
//             first product gathered from the tokens' activations:  act = silu(x Wg_e^T) .* (x Wu_e^T), then
//             y = act Wd_e^T in float32.  Every output adds its K products in the order k = 0 .. K-1 in float32,
//             so a token's result does not depend on which other tokens share its tile.
//   combine   out[token] = sum_j weight_j y[row of (token, j)]  (+ shared gate * shared expert's result), j in
//             the order of the choice.
// A second kind of router (`kind` 1): z = R x + bias (the `correction` operand), the `top` largest z are chosen (ties to
// the lower index) and their weights are the softmax over the chosen z alone; no groups.  A second shape of the gate
// (`gated` 2): g <- min(g, limit), u <- clamp(u, -limit, limit) where limit > 0, then g * sigmoid(alpha g) * (u + up_offset).
#include "common.cuh"

namespace {

constexpr int kRouteThreads = 1024;     // the most: a warp per expert for up to 32 of them at once (steps of few rows); else 256
constexpr int kMaxExperts = 1024;
constexpr int kMaxTop = 32;
constexpr int kTileRows = 32;     // rows of one expert per block of a product
constexpr int kTileCols = 64;
constexpr int kTileK = 16;

// What the two products of a gated expert become.  kind 1: silu(g) * u.  kind 2: see the head of this file.
struct ExpertGate {
    int kind;
    float alpha, limit, up_offset;
};
__device__ __forceinline__ float expert_gate(float g, float u, const ExpertGate& shape) {
    if (shape.kind == 2) {
        if (shape.limit > 0.0f) {
            g = fminf(g, shape.limit);
            u = fminf(fmaxf(u, -shape.limit), shape.limit);
        }
        return g / (1.0f + expf(-shape.alpha * g)) * (u + shape.up_offset);
    }
    return g / (1.0f + expf(-g)) * u;
}

template <typename T>
__global__ void __launch_bounds__(kRouteThreads) route_kernel(const T* x, long long ld, const float* router, const float* correction,
                                                              int width, int experts, int groups, int keep, int top, int has_gate,
                                                              int* chosen, float* weights, int* place, int* counts, float* shared_gate, int kind) {
    mlr_grid_wait();
    extern __shared__ __align__(16) float shared[];
    float* xs = shared;                 // [width]
    float* score = xs + width;          // [experts] plain scores
    float* choice = score + experts;    // [experts] scores with the correction (minus infinity once taken or not allowed)
    float* group_score = choice + experts;   // [groups]
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* xrow = x + static_cast<size_t>(row) * ld;
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = mlr_load(xrow, c);
    __syncthreads();
    for (int e = warp; e < experts + has_gate; e += warps) {
        const float* w = router + static_cast<size_t>(e) * width;
        float sum = 0.0f;
        if (width % 4 == 0) {         // 16 bytes at a time (rows of the router and the shared row start on 16-byte borders then)
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 4
            for (int c = lane; c < width / 4; c += 32) {
                const float4 a = w4[c], b = x4[c];
                sum = fmaf(a.x, b.x, sum);
                sum = fmaf(a.y, b.y, sum);
                sum = fmaf(a.z, b.z, sum);
                sum = fmaf(a.w, b.w, sum);
            }
        } else {
            for (int c = lane; c < width; c += 32) sum = fmaf(w[c], xs[c], sum);
        }
        sum = mlr_warp_sum(sum);
        if (lane == 0) {
            const float s = 1.0f / (1.0f + expf(-sum));
            if (e >= experts) {
                shared_gate[row] = s;
            } else if (kind == 1) {
                score[e] = choice[e] = sum + (correction ? correction[e] : 0.0f);
            } else {
                score[e] = s;
                choice[e] = s + (correction ? correction[e] : 0.0f);
            }
        }
    }
    __syncthreads();
    __shared__ int taken[kMaxTop];
    __shared__ float picked[kMaxTop];
    __shared__ float total_score;
    if (threadIdx.x == 0) {
    const float none = -INFINITY;
    const int per = experts / groups;
    if (groups > 1 && keep < groups) {
        for (int g = 0; g < groups; ++g) {
            float a = none, b = none;           // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = choice[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            group_score[g] = per > 1 ? a + b : a;
        }
        // Groups outside the `keep` best lose their experts: mark the kept ones by taking them out of group_score.
        for (int k = 0; k < keep; ++k) {
            int best = -1;
            float value = none;
            for (int g = 0; g < groups; ++g)
                if (!isnan(group_score[g]) && (best < 0 || group_score[g] > value)) { best = g; value = group_score[g]; }
            group_score[best] = NAN;            // NaN marks a kept group
        }
        for (int g = 0; g < groups; ++g)
            if (!isnan(group_score[g]))
                for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = none;
    }
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        int best = 0;
        float value = none;
        bool found = false;
        for (int e = 0; e < experts; ++e)
            if (!isnan(choice[e]) && (!found || choice[e] > value)) { best = e; value = choice[e]; found = true; }
        choice[best] = NAN;                     // NaN marks a taken expert
        taken[k] = best;
        picked[k] = score[best];
        total += score[best];
    }
    if (kind == 1) {
        // softmax over the chosen logits alone; the first chosen is the largest
        const float largest = picked[0];
        total = 0.0f;
        for (int k = 0; k < top; ++k) {
            picked[k] = expf(picked[k] - largest);
            total += picked[k];
        }
    }
    total_score = total;
    }
    __syncthreads();
    // One thread per chosen expert: the counters' answers come back side by side.
    if (threadIdx.x < top) {
        const int k = threadIdx.x;
        chosen[static_cast<size_t>(row) * top + k] = taken[k];
        weights[static_cast<size_t>(row) * top + k] = picked[k] / (total_score + 1e-20f);
        place[static_cast<size_t>(row) * top + k] = atomicAdd(counts + taken[k], 1);
    }
}

// One block.  first_row [experts + 1]; tiles: {expert, first row, rows} per tile, n_tiles[0] their number; row_of_pair [pairs]
// (the row of pair = token * top + choice in the order by expert), pair_of_row [pairs] the other way.
__global__ void __launch_bounds__(1024) arrange_kernel(int* counts, const int* chosen, const int* place, int experts, int pairs, int tile_rows,
                                                       int* first_row, int* tiles, int* n_tiles, int* row_of_pair, int* pair_of_row) {
    mlr_grid_wait();
    __shared__ int first[kMaxExperts + 1];
    __shared__ int first_tile[kMaxExperts + 1];
    if (threadIdx.x == 0) {
        int rows = 0, t = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = rows;
            first_tile[e] = t;
            rows += counts[e];
            t += (counts[e] + tile_rows - 1) / tile_rows;
        }
        first[experts] = rows;
        first_tile[experts] = t;
        n_tiles[0] = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) first_row[e] = first[e];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int n = first[e + 1] - first[e];
        for (int t = first_tile[e], r = 0; r < n; ++t, r += tile_rows) {
            tiles[3 * t] = e;
            tiles[3 * t + 1] = first[e] + r;
            tiles[3 * t + 2] = min(tile_rows, n - r);
        }
        counts[e] = 0;
    }
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int row = first[chosen[p]] + place[p];
        row_of_pair[p] = row;
        pair_of_row[row] = p;
    }
}

// C tile = A tile (rows of one expert, gathered through `source` / divisor when given) times W_e^T, W_e [N, K] at w + e * N * K.
// DUAL: two matrices (gate and up) and out = silu(gate) * up in TO; else the product itself in TO.
template <typename T, typename TO, bool DUAL>
__global__ void __launch_bounds__(256) expert_product_kernel(const T* a, long long lda, const int* source, int divisor, const T* w, const T* w2,
                                                             int N, int K, TO* out, long long ldo, const int* tiles, const int* n_tiles, ExpertGate shape) {
    mlr_grid_wait();
    const int tile = blockIdx.y;
    if (tile >= __ldcg(n_tiles)) return;
    const int expert = __ldcg(tiles + 3 * tile), row0 = __ldcg(tiles + 3 * tile + 1), rows = __ldcg(tiles + 3 * tile + 2);
    const int col0 = blockIdx.x * kTileCols;
    __shared__ float As[kTileK][kTileRows + 1];
    __shared__ float Ws[kTileK][kTileCols + 1];
    __shared__ float W2s[DUAL ? kTileK : 1][kTileCols + 1];
    __shared__ long long arow[kTileRows];
    if (threadIdx.x < kTileRows) {
        const int r = row0 + min(static_cast<int>(threadIdx.x), rows - 1);
        arow[threadIdx.x] = static_cast<long long>(source ? __ldcg(source + r) / divisor : r) * lda;
    }
    __syncthreads();
    const T* we = w + static_cast<size_t>(expert) * N * K;
    const T* we2 = DUAL ? w2 + static_cast<size_t>(expert) * N * K : nullptr;
    // 256 threads: thread (ty, tx) = (threadIdx.x / 16, threadIdx.x % 16) owns rows ty * 2 + {0, 1} and columns tx + 16 * {0..3}.
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[2][4] = {}, acc2[DUAL ? 2 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += kTileK) {
        for (int i = threadIdx.x; i < kTileRows * kTileK; i += 256) {
            const int r = i / kTileK, k = i % kTileK;
            As[k][r] = k0 + k < K ? mlr_load(a + arow[r], k0 + k) : 0.0f;
        }
        for (int i = threadIdx.x; i < kTileCols * kTileK; i += 256) {
            const int c = i / kTileK, k = i % kTileK;
            const bool in = col0 + c < N && k0 + k < K;
            Ws[k][c] = in ? mlr_load(we, static_cast<size_t>(col0 + c) * K + k0 + k) : 0.0f;
            if (DUAL) W2s[k][c] = in ? mlr_load(we2, static_cast<size_t>(col0 + c) * K + k0 + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTileK; ++k) {
            const float a0 = As[k][2 * ty], a1 = As[k][2 * ty + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Ws[k][tx + 16 * j];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
                if (DUAL) {
                    const float b2 = W2s[k][tx + 16 * j];
                    acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
                    acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
                }
            }
        }
        __syncthreads();
    }
    mlr_grid_dependents_may_start();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
        if (r >= rows) continue;
        TO* orow = out + static_cast<size_t>(row0 + r) * ldo;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx + 16 * j;
            if (c >= N) continue;
            float value = acc[i][j];
            if (DUAL) value = expert_gate(value, acc2[i][j], shape);
            mlr_store(orow, c, value);
        }
    }
}

// Tiles of 64 rows: stages and values of K a stage.  Measured on 8192 rows of 16 experts of 1024 x 2048 (gate/up, down):
// 3 x 32: 306 / 155 us, 4 x 32: 299 / 154 us, 2 x 64: 252 / 136 us, 3 x 64 (one block an SM): 342 / 158 us; all give the same bits.
#ifndef MLR_WIDE_STAGES
#define MLR_WIDE_STAGES 2
#define MLR_WIDE_K 64
#endif
// ---- the same product on the tensor cores (bfloat16 operands, float32 sums) ----
// A block owns a tile of 32 or 64 rows x 128 columns: 8 warps as 2 x 4, a warp 16 or 32 rows x 32 columns (four n8 pieces, and as
// many again for the second matrix when DUAL).  Rows of A (gathered) and of W arrive 32 or 64 values of K at a time by asynchronous
// 16-byte copies into one of several stages while another is multiplied; fragments by ldmatrix from rows padded by 16 bytes.
// A sum runs over K in the order of the instruction's own tree within 16 values and k = 0, 16, 32 .. between them, whatever
// else is in the tile.
constexpr int kMmaCols = 128;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

// Stages of the copy pipeline: a tile of 32 rows belongs to a step of few rows, whose blocks are fewer than the SMs and wait
// for memory: five stages of 32 values of K keep more bytes in flight; tiles of 64 rows take two stages of 64 values, which
// leaves room for two blocks an SM and halves the meetings of the block per value of K.
__host__ __device__ constexpr int mma_stages(int bm) { return bm == 32 ? 5 : MLR_WIDE_STAGES; }
// Values of K a stage holds, and the stride of a staged row (16 bytes of padding keep ldmatrix off bank conflicts).
__host__ __device__ constexpr int mma_k(int bm) { return bm == 32 ? 32 : MLR_WIDE_K; }
__host__ __device__ constexpr int mma_ld(int bm) { return mma_k(bm) + 8; }
constexpr size_t mma_shared_bytes(int bm, bool dual) { return sizeof(__nv_bfloat16) * mma_stages(bm) * (bm + (dual ? 2 : 1) * kMmaCols) * mma_ld(bm); }

// BM: rows of a tile.  8 warps as 2 x 4; a warp owns 16 x 32 of a 32-row tile and 32 x 32 of a 64-row tile (every fragment of W then
// serves two fragments of A).
template <typename TO, bool DUAL, int BM>
__global__ void __launch_bounds__(256) expert_product_mma_kernel(const __nv_bfloat16* a, long long lda, const int* source, int divisor,
                                                                 const __nv_bfloat16* w, const __nv_bfloat16* w2, int N, int K, TO* out,
                                                                 long long ldo, const int* tiles, const int* n_tiles, int all_rows,
                                                                 int a_step, int out_step, ExpertGate shape) {
    mlr_grid_wait();
    // With a tile list: tile blockIdx.y of it.  Without: every matrix (blockIdx.z) takes all `all_rows` rows, its inputs `a_step`
    // columns and its outputs `out_step` columns further right than those of the matrix before.
    constexpr int kMmaStages = mma_stages(BM), kMmaK = mma_k(BM), kMmaLd = mma_ld(BM), kChunks = kMmaK / 8;
    int expert, row0, rows;
    if (tiles) {
        const int tile = blockIdx.y;
        if (tile >= __ldcg(n_tiles)) return;
        expert = __ldcg(tiles + 3 * tile), row0 = __ldcg(tiles + 3 * tile + 1), rows = __ldcg(tiles + 3 * tile + 2);
    } else {
        expert = blockIdx.z, row0 = blockIdx.y * BM, rows = min(BM, all_rows - row0);
        a += static_cast<size_t>(expert) * a_step;
        out += static_cast<size_t>(expert) * out_step;
    }
    const int col0 = blockIdx.x * kMmaCols;
    constexpr int WN = 4;                             // warps across the columns
    constexpr int NP = kMmaCols / WN / 8;             // n8 pieces of a warp
    constexpr int MT = BM / 32;                       // m16 pieces of a warp
    constexpr int kStage = (BM + (DUAL ? 2 : 1) * kMmaCols) * kMmaLd;
    extern __shared__ __align__(16) __nv_bfloat16 staged[];       // per stage: A [BM][kMmaLd], W [128][kMmaLd], W2 the same
    __shared__ long long arow[BM];
    if (threadIdx.x < BM) {
        const int r = row0 + min(static_cast<int>(threadIdx.x), rows - 1);
        arow[threadIdx.x] = static_cast<long long>(source ? __ldcg(source + r) / divisor : r) * lda;
    }
    __syncthreads();
    const __nv_bfloat16* we = w + static_cast<size_t>(expert) * N * K;
    const __nv_bfloat16* we2 = DUAL ? w2 + static_cast<size_t>(expert) * N * K : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp / WN, wn = warp % WN;
    const int steps = (K + kMmaK - 1) / kMmaK;
    auto fetch = [&](int step, int stage) {
        if (step < steps) {
            const int k0 = step * kMmaK;
            __nv_bfloat16* As = staged + stage * kStage;
            __nv_bfloat16* Ws = As + BM * kMmaLd;
            __nv_bfloat16* W2s = Ws + kMmaCols * kMmaLd;
#pragma unroll
            for (int i = threadIdx.x; i < BM * kChunks; i += 256) {
                const int r = i / kChunks, c = (i % kChunks) * 8, k = k0 + c;
                mlr_async_copy16(&As[r * kMmaLd + c], k < K ? a + arow[r] + k : a, k < K);
            }
#pragma unroll
            for (int i = threadIdx.x; i < kMmaCols * kChunks; i += 256) {
                const int n = i / kChunks, c = (i % kChunks) * 8, k = k0 + c;
                const bool real = col0 + n < N && k < K;
                const size_t at = static_cast<size_t>(col0 + n) * K + k;
                mlr_async_copy16(&Ws[n * kMmaLd + c], real ? we + at : we, real);
                if (DUAL) mlr_async_copy16(&W2s[n * kMmaLd + c], real ? we2 + at : we2, real);
            }
        }
        mlr_async_commit();
    };
    float acc[MT][NP][4] = {}, acc2[DUAL ? MT : 1][DUAL ? NP : 1][4] = {};
#pragma unroll
    for (int st = 0; st < kMmaStages - 1; ++st) fetch(st, st);
    // ldmatrix addresses of this lane: A rows (lane & 15) at k (lane >> 4) * 8; W rows n = (lane & 7) + (lane >> 4) * 8 at k ((lane >> 3) & 1) * 8.
    const int a_off = (wm * 16 * MT + (lane & 15)) * kMmaLd + (lane >> 4) * 8;
    const int b_off = (wn * NP * 8 + (lane & 7) + (lane >> 4) * 8) * kMmaLd + ((lane >> 3) & 1) * 8;
    for (int step = 0; step < steps; ++step) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kMmaStages - 2) : "memory");
        __syncthreads();          // this step's stage has landed for everyone, and everyone is done with the stage fetched next
        fetch(step + kMmaStages - 1, (step + kMmaStages - 1) % kMmaStages);
        const __nv_bfloat16* As = staged + (step % kMmaStages) * kStage;
        const uint32_t a_base = static_cast<uint32_t>(__cvta_generic_to_shared(As));
        const uint32_t b_base = a_base + 2 * BM * kMmaLd;
        const uint32_t b2_base = b_base + 2 * kMmaCols * kMmaLd;
#pragma unroll
        for (int ks = 0; ks < kMmaK / 16; ++ks) {
            uint32_t fa[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(fa[mt], a_base + 2 * (a_off + mt * 16 * kMmaLd + ks * 16));
#pragma unroll
            for (int pair = 0; pair < NP / 2; ++pair) {
                uint32_t fb[4];
                ldmatrix_x4(fb, b_base + 2 * (b_off + pair * 16 * kMmaLd + ks * 16));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16(acc[mt][2 * pair], fa[mt], fb[0], fb[1]);
                    mma_bf16(acc[mt][2 * pair + 1], fa[mt], fb[2], fb[3]);
                }
                if (DUAL) {
                    ldmatrix_x4(fb, b2_base + 2 * (b_off + pair * 16 * kMmaLd + ks * 16));
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_bf16(acc2[mt][2 * pair], fa[mt], fb[0], fb[1]);
                        mma_bf16(acc2[mt][2 * pair + 1], fa[mt], fb[2], fb[3]);
                    }
                }
            }
        }
    }
    mlr_async_wait();
    mlr_grid_dependents_may_start();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int piece = 0; piece < NP; ++piece)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 16 * MT + mt * 16 + (lane >> 2) + 8 * half;
            const int c = col0 + wn * NP * 8 + piece * 8 + (lane & 3) * 2;
            if (r >= rows) continue;
            TO* orow = out + static_cast<size_t>(row0 + r) * ldo;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (c + j >= N) continue;
                float value = acc[mt][piece][2 * half + j];
                if (DUAL) value = expert_gate(value, acc2[DUAL ? mt : 0][DUAL ? piece : 0][2 * half + j], shape);
                mlr_store(orow, c + j, value);
            }
        }
}

template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const float* y, long long ldy, const int* row_of_pair, const float* weights, int top,
                                                      const T* shared_y, long long ld_shared, const float* shared_gate, float* out,
                                                      long long ldo, int width) {
    mlr_grid_wait();
    const int row = blockIdx.x;
    __shared__ float weight[kMaxTop];
    __shared__ long long from[kMaxTop];
    if (threadIdx.x < top) {
        weight[threadIdx.x] = __ldcg(weights + row * top + threadIdx.x);
        from[threadIdx.x] = static_cast<long long>(__ldcg(row_of_pair + row * top + threadIdx.x)) * ldy;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += 256) {
        float sum = 0.0f;
#pragma unroll 4
        for (int j = 0; j < top; ++j) sum = fmaf(weight[j], __ldcg(y + from[j] + c), sum);
        if (shared_y) {
            const float v = mlr_load(shared_y + static_cast<size_t>(row) * ld_shared, c);
            sum = shared_gate ? fmaf(__ldcg(shared_gate + row), v, sum) : sum + v;
        }
        out[static_cast<size_t>(row) * ldo + c] = sum;
    }
    mlr_grid_dependents_may_start();
}

}  // namespace

// router: float32 [experts (+ 1 with has_gate), width]; correction: float32 [experts] or null; counts: int32 [experts], zero before
// the call (`mlr_experts_arrange` zeroes them again).  chosen, place: int32 [rows, top]; weights: float32 [rows, top]; shared_gate [rows].
MLR_API int mlr_experts_route(const void* x, long long ld, int act_bf16, const float* router, const float* correction, int rows, int width,
                              int experts, int groups, int keep, int top, int has_gate, int* chosen, float* weights, int* place, int* counts,
                              float* shared_gate, int kind, cudaStream_t stream) {
    MLR_REQUIRE(kind == 0 || (kind == 1 && groups == 1), "experts_route: unknown kind of router %d (or one that has no groups)", kind);
    MLR_REQUIRE(x && router && chosen && weights && place && counts && width > 0, "experts_route: bad arguments");
    MLR_REQUIRE(experts >= 1 && experts <= kMaxExperts && top >= 1 && top <= kMaxTop && top <= experts, "experts_route: %d of %d experts (at most %d of %d)",
                top, experts, kMaxTop, kMaxExperts);
    MLR_REQUIRE(groups >= 1 && experts % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (experts / groups),
                "experts_route: %d experts in %d groups of which %d are kept cannot give %d", experts, groups, keep, top);
    MLR_REQUIRE(!has_gate || shared_gate, "experts_route: no room for the shared expert's gate");
    if (rows <= 0) return 0;
    const size_t shared = sizeof(float) * (static_cast<size_t>(width) + 2 * experts + groups);
    MLR_REQUIRE(shared <= 200 * 1024, "experts_route: a row of %d values and %d experts do not fit shared memory", width, experts);
    // Few rows: few blocks, each with a warp per expert.  Many rows: the SMs are full anyway, and smaller blocks waste fewer warps.
    const int threads = rows <= 64 ? kRouteThreads : 256;
    if (act_bf16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((route_kernel<__nv_bfloat16>), dim3(rows), dim3(threads), shared, stream, static_cast<const __nv_bfloat16*>(x), ld, router,
                   correction, width, experts, groups, keep, top, has_gate, chosen, weights, place, counts, shared_gate, kind);
    } else {
        if (shared > 48 * 1024) cudaFuncSetAttribute(route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((route_kernel<float>), dim3(rows), dim3(threads), shared, stream, static_cast<const float*>(x), ld, router, correction, width,
                   experts, groups, keep, top, has_gate, chosen, weights, place, counts, shared_gate, kind);
    }
    return mlr_launched("experts_route");
}

// tiles: int32 [3 * (pairs / 32 + experts)]; first_row: int32 [experts + 1]; n_tiles: int32 [1]; row_of_pair, pair_of_row: int32 [pairs].
// tile_rows: 32, or 64 (the tensor-core products of many rows; the products must be told the same).
MLR_API int mlr_experts_arrange(int* counts, const int* chosen, const int* place, int experts, int rows, int top, int tile_rows, int* first_row,
                                int* tiles, int* n_tiles, int* row_of_pair, int* pair_of_row, cudaStream_t stream) {
    MLR_REQUIRE(tile_rows == 32 || tile_rows == 64, "experts_arrange: tiles of 32 or 64 rows, not %d", tile_rows);
    MLR_REQUIRE(counts && chosen && place && first_row && tiles && n_tiles && row_of_pair && pair_of_row && experts >= 1 && experts <= kMaxExperts,
                "experts_arrange: bad arguments");
    if (rows <= 0) return 0;
    mlr_launch(arrange_kernel, dim3(1), dim3(1024), 0, stream, counts, chosen, place, experts, rows * top, tile_rows, first_row, tiles, n_tiles,
               row_of_pair, pair_of_row);
    return mlr_launched("experts_arrange");
}

// MLR_EXPERTS_SIMT=1 keeps the bfloat16 products on the CUDA cores (for comparing the two kernels).
static bool mlr_experts_simt_only() {
    static const bool only = [] {
        const char* v = getenv("MLR_EXPERTS_SIMT");
        return v && v[0] == '1';
    }();
    return only;
}

// The most tiles `pairs` rows of `experts` experts can make (the size of the grid, and of `tiles` / 3), whichever the tile's rows.
MLR_API int mlr_experts_max_tiles(int pairs, int experts) { return pairs / kTileRows + experts; }

// Whether the tensor-core product takes these sizes (bfloat16 activations with rows of K values on 16-byte borders): 1 yes, 0 no.
MLR_API int mlr_experts_tensor_cores(int K, long long lda) { return K % 8 == 0 && lda % 8 == 0 && !mlr_experts_simt_only(); }

// a: [*, K] activations (bfloat16 or float32), row r of the product is row source[r] / divisor of `a` (or r without `source`).
// w (and w2 when `gated`): [experts, N, K] in the activations' precision.  out: [pairs, N]; float32 when out_f32, else the
// activations' precision; with `gated` 1 out = silu(a w^T) * (a w2^T), with `gated` 2 the clamped shape of alpha, limit and
// up_offset (see the head of this file).  The product has rows * top rows.
MLR_API int mlr_experts_product(const void* a, long long lda, int act_bf16, const int* source, int divisor, const void* w, const void* w2, int gated,
                                int N, int K, void* out, long long ldo, int out_f32, const int* tiles, const int* n_tiles, int rows, int top, int experts,
                                int tile_rows, float alpha, float limit, float up_offset, cudaStream_t stream) {
    const int pairs = rows * top;
    MLR_REQUIRE(gated >= 0 && gated <= 2, "experts_product: unknown gate %d", gated);
    const ExpertGate shape = {gated, alpha, limit, up_offset};
    MLR_REQUIRE(a && w && out && tiles && n_tiles && N > 0 && K > 0 && (!gated || w2) && (!source || divisor > 0), "experts_product: bad arguments");
    const bool tensor_cores = act_bf16 && K % 8 == 0 && lda % 8 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
                              reinterpret_cast<uintptr_t>(w) % 16 == 0 && (!gated || reinterpret_cast<uintptr_t>(w2) % 16 == 0) && !mlr_experts_simt_only();
    MLR_REQUIRE(tile_rows == 32 || (tile_rows == 64 && tensor_cores), "experts_product: tiles of %d rows are not built for this product", tile_rows);
    if (pairs <= 0) return 0;
    const int max_tiles = mlr_experts_max_tiles(pairs, experts);
    MLR_REQUIRE(max_tiles <= 65535, "experts_product: %d row tiles are more than a grid takes", max_tiles);
    const dim3 grid((N + kTileCols - 1) / kTileCols, max_tiles);
    // bfloat16 rows that start on 16-byte borders go to the tensor cores.
    if (tensor_cores) {
        const dim3 wide((N + kMmaCols - 1) / kMmaCols, max_tiles);
        const __nv_bfloat16 *ab = static_cast<const __nv_bfloat16*>(a), *wb = static_cast<const __nv_bfloat16*>(w),
                            *w2b = static_cast<const __nv_bfloat16*>(w2);
#define MLR_MMA(TO, DUAL, BM)                                                                                                              \
    do {                                                                                                                                   \
        cudaFuncSetAttribute(expert_product_mma_kernel<TO, DUAL, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize,                         \
                             static_cast<int>(mma_shared_bytes(BM, DUAL)));                                                                \
        mlr_launch((expert_product_mma_kernel<TO, DUAL, BM>), dim3(wide), dim3(256), mma_shared_bytes(BM, DUAL), stream, ab, lda, source,  \
                   divisor, wb, w2b, N, K, static_cast<TO*>(out), ldo, tiles, n_tiles, 0, 0, 0, shape);                                    \
    } while (0)
        if (gated && !out_f32) {
            if (tile_rows == 64) MLR_MMA(__nv_bfloat16, true, 64);
            else MLR_MMA(__nv_bfloat16, true, 32);
        } else if (!gated && out_f32) {
            if (tile_rows == 64) MLR_MMA(float, false, 64);
            else MLR_MMA(float, false, 32);
        } else {
            return mlr_fail("experts_product: this pair of precisions is not built");
        }
#undef MLR_MMA
        return mlr_launched("experts_product");
    }
#define MLR_GO(T, TO, DUAL)                                                                                                              \
    mlr_launch((expert_product_kernel<T, TO, DUAL>), dim3(grid), dim3(256), 0, stream, static_cast<const T*>(a), lda, source, divisor,   \
               static_cast<const T*>(w), static_cast<const T*>(w2), N, K, static_cast<TO*>(out), ldo, tiles, n_tiles, shape)
    if (act_bf16) {
        if (gated && !out_f32) MLR_GO(__nv_bfloat16, __nv_bfloat16, true);
        else if (!gated && out_f32) MLR_GO(__nv_bfloat16, float, false);
        else return mlr_fail("experts_product: this pair of precisions is not built");
    } else {
        if (gated) MLR_GO(float, float, true);
        else MLR_GO(float, float, false);
    }
#undef MLR_GO
    return mlr_launched("experts_product");
}

// The same tensor-core product for `count` matrices that all take the same rows (the heads of a per-head projection):
// out[m, i * N + n] = sum_k a[m, i * K + k] w[i, n, k], bfloat16 in and out.  Returns 2 (and launches nothing) for sizes it does not take.
// With a_step and out_step matrix i reads its K inputs from column i * a_step and writes its N outputs from column i * out_step.
MLR_API int mlr_batched_product_bf16_strided(const void* a, long long lda, int a_step, const void* w, void* out, long long ldo, int out_step, int rows,
                                             int count, int N, int K, cudaStream_t stream) {
    MLR_REQUIRE(a && w && out && count > 0 && count <= 65535 && N > 0 && K > 0 && a_step >= K && out_step >= N, "batched_product: bad arguments");
    if (K % 8 || lda % 8 || a_step % 8 || reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(w) % 16 || mlr_experts_simt_only()) return 2;
    if (rows <= 0) return 0;
    const __nv_bfloat16 *ab = static_cast<const __nv_bfloat16*>(a), *wb = static_cast<const __nv_bfloat16*>(w);
    const int* none = nullptr;
    if (rows > 32) {
        const dim3 grid((N + kMmaCols - 1) / kMmaCols, (rows + 63) / 64, count);
        MLR_REQUIRE(grid.y <= 65535, "batched_product: too many rows");
        cudaFuncSetAttribute(expert_product_mma_kernel<__nv_bfloat16, false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(mma_shared_bytes(64, false)));
        mlr_launch((expert_product_mma_kernel<__nv_bfloat16, false, 64>), dim3(grid), dim3(256), mma_shared_bytes(64, false), stream, ab, lda, none, 1,
                   wb, wb, N, K, static_cast<__nv_bfloat16*>(out), ldo, none, none, rows, a_step, out_step, ExpertGate{0, 0.0f, 0.0f, 0.0f});
    } else {
        const dim3 grid((N + kMmaCols - 1) / kMmaCols, 1, count);
        cudaFuncSetAttribute(expert_product_mma_kernel<__nv_bfloat16, false, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(mma_shared_bytes(32, false)));
        mlr_launch((expert_product_mma_kernel<__nv_bfloat16, false, 32>), dim3(grid), dim3(256), mma_shared_bytes(32, false), stream, ab, lda, none, 1,
                   wb, wb, N, K, static_cast<__nv_bfloat16*>(out), ldo, none, none, rows, a_step, out_step, ExpertGate{0, 0.0f, 0.0f, 0.0f});
    }
    return mlr_launched("batched_product");
}

MLR_API int mlr_batched_product_bf16(const void* a, long long lda, const void* w, void* out, long long ldo, int rows, int count, int N, int K,
                                     cudaStream_t stream) {
    return mlr_batched_product_bf16_strided(a, lda, K, w, out, ldo, N, rows, count, N, K, stream);
}

MLR_API int mlr_experts_combine(const float* y, long long ldy, const int* row_of_pair, const float* weights, int top, const void* shared_y,
                                long long ld_shared, int shared_bf16, const float* shared_gate, float* out, long long ldo, int rows, int width,
                                cudaStream_t stream) {
    MLR_REQUIRE(y && row_of_pair && weights && out && top >= 1 && width > 0, "experts_combine: bad arguments");
    if (rows <= 0) return 0;
    if (shared_bf16)
        mlr_launch((combine_kernel<__nv_bfloat16>), dim3(rows), dim3(256), 0, stream, y, ldy, row_of_pair, weights, top,
                   static_cast<const __nv_bfloat16*>(shared_y), ld_shared, shared_gate, out, ldo, width);
    else
        mlr_launch((combine_kernel<float>), dim3(rows), dim3(256), 0, stream, y, ldy, row_of_pair, weights, top,
                   static_cast<const float*>(shared_y), ld_shared, shared_gate, out, ldo, width);
    return mlr_launched("experts_combine");
}
