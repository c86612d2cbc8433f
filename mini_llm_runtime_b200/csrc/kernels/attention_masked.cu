// Attention over a paged cache whose keys and values may differ in size, with the pieces that
// vary between designs as parameters of one description (`MaskedAttentionSpec`, host memory):
//
//   which keys a query at position p sees:   j <= p,  j > p - window (window > 0),
//                                             j >= floor(p / chunk) * chunk (chunk > 0: chunks are
//                                             counted from position 0 of the sequence)
//   rotation:   the first rot_dims values of each head of q and k turned by p * freq[i], value i paired
//               with value i + rot_dims / 2; the rest pass.  Angles, cosines and sines are float32 and
//               computed from the position (no table, no largest position).
//   kept first tokens:   with a window, keys j < keep_first stay visible however far back they lie
//   score:      (q . k) * scale;  with softcap > 0 then softcap * tanh(score / softcap);  with slopes then minus
//               slopes[head] * (p - j), a bias that grows with the distance
//   sink:       softmax with exp(sink_h) added to the denominator (a key without a value whose score is a learned number
//               per head, or 0 where none is given)
//   gate:       out *= sigmoid(gate) or silu(gate), element by element (or sigmoid of ONE value per head), and a constant factor
//
// Cache of a layer: per page, the keys [kv_head][token_in_page][dim] and then the values
// [kv_head][token_in_page][vdim] (with shared_kv only the keys: a token's value is the first vdim values of its key).  `mlr_kv_rope_cache` rotates the step's keys and writes keys and
// values (`mlr_qkv_prepare_cache` first adds biases, divides heads by their root mean square and mixes in the values an earlier layer made of the same tokens); `mlr_attention_masked` rotates its query as it loads it and walks the visible keys in tiles
// of 64 with a running maximum, one block per (row, query head), so a row's result depends on its
// position and on the cache only.  Scores, weights and sums are float32; q, the cache, the gate and
// the output are float32 or bfloat16.  Keys that are not visible are never loaded.  That kernel serves
// the float32 path and sizes the others do not take.  In bfloat16, decoded tokens and short portions go to a kernel whose
// block holds all query heads of ONE kv head (the heads are the rows of its tensor-core tiles, so a range of keys is read
// once for the group), and `mlr_attention_masked_tiles` (below) takes the prompt portions in tiles of 64 rows.
#include "common.cuh"
#include <type_traits>

struct MaskedAttentionSpec {
    const float* freq;     // [rot_dims / 2] float32 on the device, or null
    const float* sinks;    // [heads] float32 on the device: the sink's score per head; null with sink set: 0
    const float* slopes;   // [heads] float32 on the device: score -= slopes[head] * distance; null: no such bias
    const float* q_weight; // the weights of a norm of q and of k that `mlr_qkv_prepare_cache` applies (float32 on the device):
    const float* k_weight; // qk_norm 1: [dim] each, shared by all heads; qk_norm 2: [heads * dim] and [kv_heads * dim]
    int heads, kv_heads, dim, vdim;
    int rot_dims, window, chunk, sink;
    int gate_kind;         // 0 none, 1 sigmoid, 2 silu, 3 sigmoid of one value per head (the gate has `heads` columns)
    int shared_kv;         // 1: a token's value is the first vdim values of its key (vdim <= dim; one vector per token is cached and a page holds keys only)
    int keep_first;        // with a window: the first keep_first positions stay visible
    int qk_norm;           // 0 none; 1 every head of q and k over its root mean square, times a weight; 2 the WHOLE projection (all heads) likewise
    int dense_cache;       // 1: `mlr_qkv_prepare_cache` serves the kernels of the plain causal attention (attention_bf16, attention_tcgen05,
                           // attention_generic) instead of this file's: it also rotates the queries in place, and writes the cache as those
                           // kernels read it ([page][K | V][kv_head][token][dim] with dim = vdim, bfloat16 rows of 64, 128 or 256 values with
                           // their 16-byte chunks swizzled by the position: `mlr_cache_col`)
    float scale, out_scale;
    float softcap;         // > 0: score <- softcap * tanh(score / softcap)
};

// What a score becomes after the product: scaled, capped, biased by the distance to the key.
__device__ __forceinline__ float mlr_masked_score(float dot, int distance, float slope, const MaskedAttentionSpec& s) {
    float score = dot * s.scale;
    if (s.softcap > 0.0f) score = s.softcap * tanhf(score / s.softcap);
    return score - slope * static_cast<float>(distance);
}

__device__ __forceinline__ float mlr_gate_value(float g, int kind) {
    const float sig = 1.0f / (1.0f + expf(-g));
    return kind == 2 ? g * sig : sig;
}

namespace {

constexpr int kTile = 64;
constexpr int kThreads = 128;
constexpr int kPrepareThreads = 1024; // the most threads of a block of `qkv_prepare_cache_kernel` (it is launched with 128 unless few rows need a whole norm)
constexpr int kMaxDimsPerThread = 8;  // vdim <= 1024; the kernels are built for 2 (vdim <= 256), 4 and 8 value columns a thread
constexpr int kRowsPerItem = 16;      // a segment that the planner gives the row kernel brings at most this many rows

// How many (row, head) results of one few-row segment the ranges' scratch holds: segments bring at most 16 / (heads per kv
// head) rows, or ONE row where more than 16 heads share a kv head.
__device__ __forceinline__ int partial_slots(const MaskedAttentionSpec& s) {
    return max(kRowsPerItem * s.kv_heads, ((s.heads + kRowsPerItem - 1) / kRowsPerItem) * kRowsPerItem);
}


template <typename T>
__global__ void __launch_bounds__(kThreads) kv_rope_cache_kernel(const T* k, int ld_k, const T* v, int ld_v, T* cache, int num_pages,
                                                                 const int* positions, const int* segment_of_row,
                                                                 const int* block_table, int table_stride, int page_size,
                                                                 MaskedAttentionSpec s, int* status) {
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int position = positions[row];
    const int page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
        return;
    }
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.shared_kv ? s.dim : s.dim + s.vdim);
    T* kbase = cache + page * page_elems + static_cast<size_t>(position % page_size) * s.dim;
    T* vbase = cache + page * page_elems + static_cast<size_t>(s.kv_heads) * page_size * s.dim +
               static_cast<size_t>(position % page_size) * s.vdim;
    const T* krow = k + static_cast<size_t>(row) * ld_k;
    const T* vrow = v + static_cast<size_t>(row) * ld_v;
    const int half = s.rot_dims / 2;
    const float p = static_cast<float>(position);
    for (int i = threadIdx.x; i < s.kv_heads * s.dim; i += kThreads) {
        const int head = i / s.dim, c = i % s.dim;
        float value = mlr_load(krow, i);
        if (c < s.rot_dims) {
            float sn, cs;
            sincosf(p * s.freq[c < half ? c : c - half], &sn, &cs);
            const float other = mlr_load(krow, c < half ? i + half : i - half);
            value = c < half ? value * cs - other * sn : value * cs + other * sn;
        }
        mlr_store(kbase + static_cast<size_t>(head) * page_size * s.dim, c, value);
    }
    for (int i = threadIdx.x; i < (s.shared_kv ? 0 : s.kv_heads * s.vdim); i += kThreads) {
        const int head = i / s.vdim, c = i % s.vdim;
        vbase[static_cast<size_t>(head) * page_size * s.vdim + c] = vrow[i];
    }
    mlr_grid_dependents_may_start();
}

// The step's q, k and v as the projection left them, made ready for attention, blocks of four warps per row and one warp per head:
//   q_h <- norm(q_h + bias)                  in place         (biases and the norm only where asked for)
//   k_g <- norm(k_g + bias), rotated like `kv_rope_cache_kernel` does, into the cache
//   v_g <- (v_g + bias) / rms(v_g);  mix 1: first[row] = v;  mix 2: v <- (1 - lambda) v + lambda first[row];  into the cache
// norm of q and k: unit_qk divides every head by its root mean square; qk_norm 1 does so and multiplies by a weight of one head's
// size that all heads share (wq, wk [dim]); qk_norm 2 divides the WHOLE projection (all heads of q, all heads of k) by its root
// mean square and multiplies by a weight of the projection's size (wq [heads * dim], wk [kv_heads * dim]; one block a row then).
// Without k (a layer that reads the keys and values another layer cached) only the queries are prepared.
// `first` is a float32 buffer of the step, [rows, kv_heads * vdim]: the values the first of several layers made of the same
// tokens, which the later ones mix into their own.  All arithmetic is float32.
template <typename T, int kBlock>
__global__ void __launch_bounds__(kBlock) qkv_prepare_cache_kernel(T* q, int ldq, const T* k, int ld_k, const T* v, int ld_v, const float* bq,
                                                                     const float* bk, const float* bv, int unit_qk, int unit_v, float eps,
                                                                     float* first, int ld_first, int mix, float lambda, T* cache, int num_pages,
                                                                     const int* positions, const int* segment_of_row, const int* block_table,
                                                                     int table_stride, int page_size, MaskedAttentionSpec s, int* status) {
    const float* wq = s.q_weight;
    const float* wk = s.k_weight;
    const int qk_norm = s.qk_norm;
    mlr_grid_wait();
    extern __shared__ __align__(16) float staged[];        // [warps][max(dim, vdim)]
    __shared__ float whole_sum[kBlock / 32];
    // kBlock: 128, or 1024 (a warp a head, launched with as many warps as there are heads) for few rows under a whole norm
    const int threads = kBlock == kThreads ? kThreads : static_cast<int>(blockDim.x), warps = threads >> 5;
    __shared__ float whole_inv[2];
    const int row = blockIdx.x;
    const int position = positions[row];
    int page = 0;
    if (k) {
        page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
            return;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* mine = staged + warp * max(s.dim, s.vdim);
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.dim + s.vdim);
    T* kbase = cache + page * page_elems + static_cast<size_t>(position % page_size) * s.dim;
    T* vbase = cache + page * page_elems + static_cast<size_t>(s.kv_heads) * page_size * s.dim +
               static_cast<size_t>(position % page_size) * s.vdim;
    const int half = s.rot_dims / 2;
    const float p = static_cast<float>(position);
    const bool swizzled = s.dense_cache && mlr_cache_swizzled(sizeof(T) == 2, s.dim);
    if (qk_norm == 2) {
        // The root mean square of a whole projection: every thread sums its columns, the warps' sums are added in order.
        for (int which = 0; which < (k ? 2 : 1); ++which) {
            const T* src = which == 0 ? q + static_cast<size_t>(row) * ldq : k + static_cast<size_t>(row) * ld_k;
            const float* bias = which == 0 ? bq : bk;
            const int total = (which == 0 ? s.heads : s.kv_heads) * s.dim;
            float squares = 0.0f;
            for (int c = threadIdx.x; c < total; c += threads) {
                const float value = mlr_load(src, c) + (bias ? bias[c] : 0.0f);
                squares = fmaf(value, value, squares);
            }
            squares = mlr_warp_sum(squares);
            if (lane == 0) whole_sum[warp] = squares;
            __syncthreads();
            if (threadIdx.x == 0) {
                float sum = 0.0f;
                for (int w = 0; w < warps; ++w) sum += whole_sum[w];
                whole_inv[which] = 1.0f / sqrtf(sum / static_cast<float>(total) + eps);
            }
            __syncthreads();
        }
    }
    const int units = k ? s.heads + 2 * s.kv_heads : s.heads;
    for (int unit = blockIdx.y * warps + warp; unit < units; unit += gridDim.y * warps) {
        const int kind = unit < s.heads ? 0 : (unit < s.heads + s.kv_heads ? 1 : 2);
        const int head = kind == 0 ? unit : (kind == 1 ? unit - s.heads : unit - s.heads - s.kv_heads);
        const int n = kind == 2 ? s.vdim : s.dim;
        const T* src = kind == 0 ? q + static_cast<size_t>(row) * ldq : (kind == 1 ? k + static_cast<size_t>(row) * ld_k : v + static_cast<size_t>(row) * ld_v);
        const float* bias = kind == 0 ? bq : (kind == 1 ? bk : bv);
        float squares = 0.0f;
        for (int c = lane; c < n; c += 32) {
            float value = mlr_load(src, static_cast<size_t>(head) * n + c);
            if (bias) value += bias[head * n + c];
            mine[c] = value;
            squares = fmaf(value, value, squares);
        }
        const bool head_norm = kind == 2 ? unit_v : (unit_qk || qk_norm == 1);
        float inv = head_norm ? 1.0f / sqrtf(mlr_warp_sum(squares) / static_cast<float>(n) + eps) : 1.0f;
        const float* weight = nullptr;
        if (kind < 2 && qk_norm == 2) {
            inv = whole_inv[kind];
            weight = (kind == 0 ? wq : wk) + static_cast<size_t>(head) * n;
        } else if (kind < 2 && qk_norm == 1) {
            weight = kind == 0 ? wq : wk;
        }
        for (int c = lane; c < n; c += 32) mine[c] = mine[c] * inv * (weight ? weight[c] : 1.0f);     // a lane's own values
        __syncwarp();
        if (kind == 0 && !s.dense_cache) {
            T* dst = q + static_cast<size_t>(row) * ldq + static_cast<size_t>(head) * n;
            for (int c = lane; c < n; c += 32) mlr_store(dst, c, mine[c]);
        } else if (kind < 2) {
            // Keys go to the cache rotated; queries are rotated here only for kernels that do not rotate them as they load them.
            T* dst = kind == 0 ? q + static_cast<size_t>(row) * ldq + static_cast<size_t>(head) * n : kbase + static_cast<size_t>(head) * page_size * s.dim;
            for (int c = lane; c < n; c += 32) {
                float value = mine[c];
                if (c < s.rot_dims) {
                    float sn, cs;
                    sincosf(p * s.freq[c < half ? c : c - half], &sn, &cs);
                    const float other = mine[c < half ? c + half : c - half];
                    value = c < half ? value * cs - other * sn : value * cs + other * sn;
                }
                mlr_store(dst, kind == 1 ? mlr_cache_col(c, position, swizzled) : c, value);
            }
        } else {
            T* dst = vbase + static_cast<size_t>(head) * page_size * s.vdim;
            float* keep = first ? first + static_cast<size_t>(row) * ld_first + static_cast<size_t>(head) * n : nullptr;
            for (int c = lane; c < n; c += 32) {
                float value = mine[c];
                if (mix == 1) keep[c] = value;
                else if (mix == 2) value = (1.0f - lambda) * value + lambda * __ldcg(keep + c);
                mlr_store(dst, mlr_cache_col(c, position, swizzled), value);
            }
        }
        __syncwarp();
    }
    mlr_grid_dependents_may_start();
}

template <typename T, int DPT>
__global__ void __launch_bounds__(kThreads) attention_masked_kernel(const T* q, int ldq, const T* gate, int ld_gate, T* out, int ldo,
                                                                    const T* cache, int num_pages, const int* positions,
                                                                    const int* segment_of_row, const int* block_table,
                                                                    int table_stride, int page_size, MaskedAttentionSpec s,
                                                                    const int* items, const int* segment_info, int split_keys,
                                                                    int max_splits, float* partial, int* status) {
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    long long* offsets = reinterpret_cast<long long*>(smem);   // [kTile] element offset of the token's value row
    float* scores = reinterpret_cast<float*>(offsets + kTile);  // [kTile]
    float* qs = scores + kTile;                                  // [dim]
    __shared__ int bad;

    // With `segment_info`, blockIdx.x names a segment of few rows (`items` lists those segments, or all are) and the block
    // walks its rows one after the other; without, blockIdx.x is the row.
    int first_row = blockIdx.x, n_rows = 1;
    if (segment_info) {
        const int* info = segment_info + 4 * (items ? items[blockIdx.x] : blockIdx.x);
        first_row = info[0];
        n_rows = min(info[1], kRowsPerItem);
    }
    const int head = blockIdx.y;
    auto one_row = [&](const int row, const int j) {
    __syncthreads();            // the row before is done with the shared memory
    const int kv_head = head / (s.heads / s.kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int position = positions[row];
    const int segment = segment_of_row[row];
    int lo = 0;
    if (s.window > 0) lo = max(lo, position - s.window + 1);
    if (s.chunk > 0) lo = max(lo, (position / s.chunk) * s.chunk);
    const int kept = (s.window > 0 && s.keep_first > 0) ? min(s.keep_first, lo) : 0;       // keys [0, kept) are seen beside [lo, position]
    const float slope = s.slopes ? s.slopes[head] : 0.0f;
    const float sink_score = s.sinks ? s.sinks[head] : 0.0f;
    const int* table = block_table + static_cast<size_t>(segment) * table_stride;
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.shared_kv ? s.dim : s.dim + s.vdim);
    const size_t key_plane = s.shared_kv ? 0 : static_cast<size_t>(s.kv_heads) * page_size * s.dim;
    const int value_row = s.shared_kv ? s.dim : s.vdim;      // values between two tokens' value rows

    const T* qrow = q + static_cast<size_t>(row) * ldq + static_cast<size_t>(head) * s.dim;
    const int half = s.rot_dims / 2;
    const float p = static_cast<float>(position);
    for (int c = threadIdx.x; c < s.dim; c += kThreads) {
        float value = mlr_load(qrow, c);
        if (c < s.rot_dims) {
            float sn, cs;
            sincosf(p * s.freq[c < half ? c : c - half], &sn, &cs);
            const float other = mlr_load(qrow, c < half ? c + half : c - half);
            value = c < half ? value * cs - other * sn : value * cs + other * sn;
        }
        qs[c] = value;
    }
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();

    // The sink is a key of score 0 that is always seen and carries no value.  With `partial` the visible keys are cut
    // into ranges of `split_keys` (from the 64-key border at or below the first one); blockIdx.z names this block's
    // range, whose maximum, sum and weighted values go to `partial` for `attention_masked_merge_kernel` (the sink too).
    float running_max = (s.sink && !partial) ? sink_score : -INFINITY, running_sum = (s.sink && !partial) ? 1.0f : 0.0f;
    float acc[DPT] = {};
    int tile_first = (lo / kTile) * kTile, tile_last = position;
    if (partial) {
        tile_first += blockIdx.z * split_keys;
        tile_last = min(position, tile_first + split_keys - 1);
        if (tile_first > position) return;           // the merge reads only the ranges that exist for this row
    }

    constexpr int kChunk = 16 / sizeof(T);                      // values in 16 bytes
    const bool chunked_rows = s.dim % kChunk == 0;              // a key's row is whole 16-byte pieces, each aligned
    // The kept first keys come first, as tiles of their own (of the first key range only); then the window's tiles.
    const int kept_tiles = (kept > 0 && (!partial || blockIdx.z == 0)) ? (kept + kTile - 1) / kTile : 0;
    const int main_tiles = (tile_last - tile_first) / kTile + 1;
    for (int step = 0; step < kept_tiles + main_tiles; ++step) {
        const bool early = step < kept_tiles;
        const int tile = early ? step * kTile : tile_first + (step - kept_tiles) * kTile;
        const int see_lo = early ? 0 : lo, see_hi = early ? kept - 1 : tile_last;
        if (chunked_rows) {
            // Scores of this tile: two threads per key, each adds up every other 16-byte piece of the key's row.
            const int i = threadIdx.x >> 1, t = tile + i;
            float partial = 0.0f;
            long long offset = -1;
            if (t >= see_lo && t <= see_hi) {
                const int page = table[t / page_size];
                if (page < 0 || page >= num_pages) {
                    bad = 1;
                } else {
                    const T* k = cache + page * page_elems + (static_cast<size_t>(kv_head) * page_size + t % page_size) * s.dim;
                    offset = static_cast<long long>(page * page_elems + key_plane +
                                                    (static_cast<size_t>(kv_head) * page_size + t % page_size) * value_row);
                    for (int c0 = (threadIdx.x & 1) * kChunk; c0 < s.dim; c0 += 8 * kChunk) {     // four pieces on their way at a time
                        float v[4][kChunk];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int c = c0 + j * 2 * kChunk;
                            if (c < s.dim) {
                                if constexpr (sizeof(T) == 2) mlr_load8(k + c, v[j]);
                                else mlr_load4(k + c, v[j]);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int c = c0 + j * 2 * kChunk;
                            if (c < s.dim) {
#pragma unroll
                                for (int e = 0; e < kChunk; ++e) partial = fmaf(qs[c + e], v[j][e], partial);
                            }
                        }
                    }
                }
            }
            partial += __shfl_xor_sync(0xffffffffu, partial, 1);
            if ((threadIdx.x & 1) == 0) {
                scores[i] = offset >= 0 ? mlr_masked_score(partial, position - t, slope, s) : -INFINITY;
                offsets[i] = offset;
            }
        } else
        for (int i = warp; i < kTile; i += kThreads / 32) {
            const int t = tile + i;
            float score = -INFINITY;
            long long offset = -1;
            if (t >= see_lo && t <= see_hi) {
                const int page = table[t / page_size];
                if (page < 0 || page >= num_pages) {
                    if (lane == 0) bad = 1;
                } else {
                    const T* k = cache + page * page_elems + (static_cast<size_t>(kv_head) * page_size + t % page_size) * s.dim;
                    offset = static_cast<long long>(page * page_elems + key_plane +
                                                    (static_cast<size_t>(kv_head) * page_size + t % page_size) * value_row);
                    float partial = 0.0f;
                    for (int j = lane; j < s.dim; j += 32) partial = fmaf(qs[j], mlr_load(k, j), partial);
                    score = mlr_masked_score(mlr_warp_sum(partial), position - t, slope, s);
                }
            }
            if (lane == 0) {
                scores[i] = score;
                offsets[i] = offset;
            }
        }
        __syncthreads();
        float tile_max = -INFINITY;
        for (int i = 0; i < kTile; ++i) tile_max = fmaxf(tile_max, scores[i]);
        const float new_max = fmaxf(running_max, tile_max);
        __syncthreads();
        if (threadIdx.x < kTile) {
            const float sc = scores[threadIdx.x];
            scores[threadIdx.x] = (sc == -INFINITY) ? 0.0f : expf(sc - new_max);
        }
        __syncthreads();
        if (new_max > -INFINITY) {
            const float alpha = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
            running_sum *= alpha;
#pragma unroll
            for (int d = 0; d < DPT; ++d) acc[d] *= alpha;
            for (int i0 = 0; i0 < kTile; i0 += 8) {       // eight keys' values are on their way before the first is used
                float values[8][DPT];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const long long offset = offsets[i0 + u];
#pragma unroll
                    for (int d = 0; d < DPT; ++d) {
                        const int c = threadIdx.x + d * kThreads;
                        values[u][d] = (offset >= 0 && c < s.vdim) ? mlr_load(cache + offset, c) : 0.0f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float w = scores[i0 + u];         // 0 for a key that is not seen
                    running_sum += w;
#pragma unroll
                    for (int d = 0; d < DPT; ++d) acc[d] = fmaf(w, values[u][d], acc[d]);
                }
            }
            running_max = new_max;
        }
        __syncthreads();
    }
    if (bad && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
    if (partial) {
        float* mine = partial + ((static_cast<size_t>(blockIdx.x) * partial_slots(s) + j * s.heads + head) * max_splits +
                                 blockIdx.z) * (s.vdim + 2);
        if (threadIdx.x == 0) {
            mine[0] = running_max;
            mine[1] = running_sum;
        }
#pragma unroll
        for (int d = 0; d < DPT; ++d) {
            const int c = threadIdx.x + d * kThreads;
            if (c < s.vdim) mine[2 + c] = acc[d];
        }
        return;
    }
    T* orow = out + static_cast<size_t>(row) * ldo + static_cast<size_t>(head) * s.vdim;
    const T* grow = gate ? gate + static_cast<size_t>(row) * ld_gate + static_cast<size_t>(head) * (s.gate_kind == 3 ? 1 : s.vdim) : nullptr;
#pragma unroll
    for (int d = 0; d < DPT; ++d) {
        const int c = threadIdx.x + d * kThreads;
        if (c < s.vdim) {
            float value = running_sum > 0.0f ? acc[d] / running_sum : 0.0f;
            if (grow) value *= mlr_gate_value(mlr_load(grow, s.gate_kind == 3 ? 0 : c), s.gate_kind);
            mlr_store(orow, c, value * s.out_scale);
        }
    }
    };
    for (int j = 0; j < n_rows; ++j) one_row(first_row + j, j);
    mlr_grid_dependents_may_start();
}

// Adds up the key ranges of every row of a segment: grid (segments of few rows, heads), as the row kernel's.
template <typename T, int DPT>
__global__ void __launch_bounds__(kThreads) attention_masked_merge_kernel(const float* partial, const T* gate, int ld_gate, T* out, int ldo,
                                                                          const int* positions, MaskedAttentionSpec s, const int* items,
                                                                          const int* segment_info, int split_keys, int max_splits) {
    mlr_grid_wait();
    const int item = blockIdx.x, head = blockIdx.y;
    const int* info = segment_info + 4 * (items ? items[item] : item);
    for (int j = 0; j < min(info[1], kRowsPerItem); ++j) {
    const int row = info[0] + j;
    const int position = positions[row];
    int lo = 0;
    if (s.window > 0) lo = max(lo, position - s.window + 1);
    if (s.chunk > 0) lo = max(lo, (position / s.chunk) * s.chunk);
    const int splits = (position - (lo / kTile) * kTile) / split_keys + 1;
    const float* mine = partial + (static_cast<size_t>(item) * partial_slots(s) + j * s.heads + head) * max_splits * (s.vdim + 2);
    const float sink_score = s.sinks ? s.sinks[head] : 0.0f;
    float top = s.sink ? sink_score : -INFINITY;
    for (int i = 0; i < splits; ++i) top = fmaxf(top, __ldcg(mine + static_cast<size_t>(i) * (s.vdim + 2)));
    float sum = s.sink ? expf(sink_score - top) : 0.0f;
    float acc[DPT] = {};
    for (int i = 0; i < splits; ++i) {
        const float* part = mine + static_cast<size_t>(i) * (s.vdim + 2);
        const float m = __ldcg(part);
        if (m == -INFINITY) continue;
        const float w = expf(m - top);
        sum = fmaf(__ldcg(part + 1), w, sum);
#pragma unroll
        for (int d = 0; d < DPT; ++d) {
            const int c = threadIdx.x + d * kThreads;
            if (c < s.vdim) acc[d] = fmaf(__ldcg(part + 2 + c), w, acc[d]);
        }
    }
    T* orow = out + static_cast<size_t>(row) * ldo + static_cast<size_t>(head) * s.vdim;
    const T* grow = gate ? gate + static_cast<size_t>(row) * ld_gate + static_cast<size_t>(head) * (s.gate_kind == 3 ? 1 : s.vdim) : nullptr;
#pragma unroll
    for (int d = 0; d < DPT; ++d) {
        const int c = threadIdx.x + d * kThreads;
        if (c < s.vdim) {
            float value = sum > 0.0f ? acc[d] / sum : 0.0f;
            if (grow) value *= mlr_gate_value(mlr_load(grow, s.gate_kind == 3 ? 0 : c), s.gate_kind);
            mlr_store(orow, c, value * s.out_scale);
        }
    }
    }
    mlr_grid_dependents_may_start();
}

// ---- prompt portions in bfloat16: 64 query rows of one request and one head per block, on the tensor cores.
// S = Q K^T by mma.sync (bfloat16 operands, float32 sums: the scores are exact products summed in float32); mask, sink
// and the running softmax in float32; the weights enter P V as TWO bfloat16 terms (p = hi + lo, 16 bits of
// mantissa) against the bfloat16 values, again with float32 sums.  Keys and values of a tile of 64 positions are
// copied from their pages into shared memory (zeros where no row of the block may look), one tile ahead.
constexpr int kRows = 64, kKeys = 64, kPad = 8;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// What a product becomes in the tensor-core kernels.  Without a cap `to_cap` = scale.  With one, `to_cap` = 2 log2(e) scale / cap
// and cap * tanh(x) = cap - 2 cap / (e^(2x) + 1), one exponential and one reciprocal of the special-function unit for either
// sign of x (e^(2x) = inf gives cap, 0 gives -cap).  Near x = 0 the difference loses relative precision, not absolute: the
// score is off by a few 2^-23 of the cap, far below what bfloat16 queries and keys leave.  `back` = key - position as a float
// (exact: both are far below 2^24), so that the distance bias is one fused multiply-add.
template <bool CAPPED>
__device__ __forceinline__ float tile_score(float dot, float back, float to_cap, float cap, float slope) {
    float v = dot * to_cap;
    if (CAPPED) {
        float e, r;
        asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(v));
        asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(e + 1.0f));
        v = fmaf(-2.0f * cap, r, cap);
    }
    return fmaf(slope, back, v);
}

__device__ __forceinline__ int first_visible(int position, const MaskedAttentionSpec& s) {
    int lo = 0;
    if (s.window > 0) lo = max(lo, position - s.window + 1);
    if (s.chunk > 0) lo = max(lo, (position / s.chunk) * s.chunk);
    return lo;
}

template <int NV>
__global__ void __launch_bounds__(128) attention_masked_tile_kernel(const __nv_bfloat16* q, int ldq, const __nv_bfloat16* gate, int ld_gate,
                                                                    __nv_bfloat16* out, int ldo, const __nv_bfloat16* cache, int num_pages,
                                                                    const int* tiles, const int* segment_info, const int* block_table,
                                                                    int table_stride, int page_size, MaskedAttentionSpec s, int* status) {
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int qstride = s.dim + kPad, vstride = s.shared_kv ? qstride : s.vdim + kPad;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* Ks = Qs + kRows * qstride;
    __nv_bfloat16* Vs = s.shared_kv ? Ks : Ks + 2 * kKeys * qstride;        // two stages of each; values that are their keys' start are read there
    __shared__ int bad;

    const int tile_index = blockIdx.y;       // the planner lists the tiles that see the most keys first
    const int head = blockIdx.x, kv_head = head / (s.heads / s.kv_heads);
    const int segment = tiles[2 * tile_index], tile_token = tiles[2 * tile_index + 1];
    const int first = segment_info[4 * segment], count = segment_info[4 * segment + 1], start = segment_info[4 * segment + 2];
    const int n_rows = min(kRows, count - tile_token);
    const int first_pos = start + tile_token, last_pos = first_pos + n_rows - 1;
    const int lo_min = first_visible(first_pos, s);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int* table = block_table + static_cast<size_t>(segment) * table_stride;
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.shared_kv ? s.dim : s.dim + s.vdim);
    const size_t key_plane = s.shared_kv ? 0 : static_cast<size_t>(s.kv_heads) * page_size * s.dim;
    const int value_row = s.shared_kv ? s.dim : s.vdim;
    const int keep_first = s.window > 0 ? s.keep_first : 0;
    const float slope = s.slopes ? s.slopes[head] : 0.0f;
    const float sink_score = s.sinks ? s.sinks[head] : 0.0f;
    const bool capped = s.softcap > 0.0f, plain_scores = !capped && !s.slopes;
    const float to_cap = capped ? 2.0f * 1.4426950408889634f * s.scale / s.softcap : s.scale;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();

    // The block's queries, rotated in float32, as bfloat16.
    const int half = s.rot_dims / 2;
    for (int i = threadIdx.x; i < kRows * s.dim; i += 128) {
        const int r = i / s.dim, c = i % s.dim;
        float value = 0.0f;
        if (r < n_rows) {
            const __nv_bfloat16* qrow = q + static_cast<size_t>(first + tile_token + r) * ldq + static_cast<size_t>(head) * s.dim;
            value = __bfloat162float(qrow[c]);
            if (c < s.rot_dims) {
                float sn, cs;
                sincosf(static_cast<float>(first_pos + r) * s.freq[c < half ? c : c - half], &sn, &cs);
                const float other = __bfloat162float(qrow[c < half ? c + half : c - half]);
                value = c < half ? value * cs - other * sn : value * cs + other * sn;
            }
        }
        Qs[r * qstride + c] = __float2bfloat16_rn(value);
    }

    const int r0 = warp * 16;
    const int pos_a = first_pos + r0 + g, pos_b = pos_a + 8;         // this thread's two rows
    const bool row_a = r0 + g < n_rows, row_b = r0 + g + 8 < n_rows;
    const int lo_a = first_visible(pos_a, s), lo_b = first_visible(pos_b, s);
    float m_a = s.sink ? sink_score : -INFINITY, m_b = m_a, l_a = s.sink ? 1.0f : 0.0f, l_b = l_a;   // l: this thread's share, but the sink's 1
    if (t != 0) l_a = l_b = 0.0f;                                                                // is counted once per row
    float O[NV][4];
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) O[nv][0] = O[nv][1] = O[nv][2] = O[nv][3] = 0.0f;
    const int ksteps = s.dim / 16;
    const uint32_t vs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vs));
    const uint32_t qs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Qs));
    const uint32_t ks_base = static_cast<uint32_t>(__cvta_generic_to_shared(Ks));

    // Keys and values of a tile of 64 positions go from their pages into one of two stages by asynchronous copies, so
    // that the next tile arrives while this one is multiplied; rows no query of the block may see become zeros.
    // The page of this thread's key of the tile at `kt` (0 where no query of the block sees the key).  It is read one tile
    // before the copies that need it are issued, so that no warp waits for the table between two tiles.
    auto page_for = [&](int kt) {
        const int position = kt + (threadIdx.x >> 1);
        const bool real = position <= last_pos && (position >= lo_min || position < keep_first);
        return real ? __ldg(table + position / page_size) : 0;
    };
    auto fetch = [&](int kt, int into, int page) {
        __nv_bfloat16* kdst = Ks + into * kKeys * qstride;
        __nv_bfloat16* vdst = Vs + into * kKeys * vstride;
        // Two threads per key: the row's addresses once, then every other 16-byte piece of the key's row and of its value row.
        const int key = threadIdx.x >> 1, position = kt + key;
        bool real = position <= last_pos && (position >= lo_min || position < keep_first);
        const __nv_bfloat16* ksrc = cache;
        const __nv_bfloat16* vsrc = cache;
        if (real) {
            if (page < 0 || page >= num_pages) {
                bad = 1;
                real = false;
            } else {
                const size_t in_page = static_cast<size_t>(kv_head) * page_size + position % page_size;
                ksrc = cache + page * page_elems + in_page * s.dim;
                vsrc = cache + page * page_elems + key_plane + in_page * value_row;
            }
        }
        __nv_bfloat16* krow = kdst + key * qstride;
        __nv_bfloat16* vrow = vdst + key * vstride;
        for (int c = (threadIdx.x & 1) * 8; c < s.dim; c += 16) mlr_async_copy16(krow + c, real ? ksrc + c : cache, real);
        if (!s.shared_kv)
            for (int c = (threadIdx.x & 1) * 8; c < s.vdim; c += 16) mlr_async_copy16(vrow + c, real ? vsrc + c : cache, real);
        mlr_async_commit();
    };
    // Tiles of keys in the order they are walked: those of the kept first tokens that lie before the window's first tile, then
    // the window's tiles up to the block's last position.
    const int kt_first = (lo_min / kKeys) * kKeys;
    const int early_tiles = (min(keep_first, kt_first) + kKeys - 1) / kKeys;
    const int all_tiles = early_tiles + (last_pos - kt_first) / kKeys + 1;
    auto tile_start = [&](int i) { return i < early_tiles ? i * kKeys : kt_first + (i - early_tiles) * kKeys; };
    fetch(tile_start(0), 0, page_for(tile_start(0)));
    int page_ahead = all_tiles > 1 ? page_for(tile_start(1)) : 0;
    int current = 0;
    for (int ti = 0; ti < all_tiles; ++ti, current ^= 1) {
        const int kt = tile_start(ti);
        mlr_async_wait();
        __syncthreads();      // this tile has arrived (and Qs is written); no warp still reads the other stage
        if (ti + 1 < all_tiles) {
            fetch(tile_start(ti + 1), current ^ 1, page_ahead);
            if (ti + 2 < all_tiles) page_ahead = page_for(tile_start(ti + 2));
        }
        const uint32_t kt_base = ks_base + static_cast<uint32_t>(current * kKeys * qstride * 2);
        const uint32_t vt_base = vs_base + static_cast<uint32_t>(current * kKeys * vstride * 2);
        float S[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.0f;
        // Fragments by ldmatrix: one x4 gives the 16 x 16 piece of Q; one x4 gives, for 8 keys, the pieces of two
        // steps of 16 along the head (a last odd step takes an x2).
        const uint32_t q_row = qs_base + static_cast<uint32_t>(((r0 + (lane & 7) + ((lane >> 3) & 1) * 8) * qstride + (lane >> 4) * 8) * 2);
        const uint32_t k_row = kt_base + static_cast<uint32_t>((((lane & 7)) * qstride + (lane >> 3) * 8) * 2);
        for (int ks = 0; ks < ksteps; ks += 2) {
            uint32_t a[4], a2[4] = {0, 0, 0, 0};
            ldmatrix_x4(a, q_row + ks * 32);
            const bool two = ks + 1 < ksteps;
            if (two) ldmatrix_x4(a2, q_row + (ks + 1) * 32);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint32_t kb[4];
                const uint32_t at = k_row + static_cast<uint32_t>((nt * 8 * qstride + ks * 16) * 2);
                if (two) {
                    ldmatrix_x4(kb, at);
                    mma_bf16(S[nt], a, kb[0], kb[1]);
                    mma_bf16(S[nt], a2, kb[2], kb[3]);
                } else {
                    ldmatrix_x2(kb, at);
                    mma_bf16(S[nt], a, kb[0], kb[1]);
                }
            }
        }
        // mask, running maximum.  A tile whose 64 keys every one of the warp's 16 rows sees needs no mask (the same for
        // all lanes of a warp): all rows exist, the last key is at or before the first row, the first key at or after
        // the last row's first visible one.
        float tile_a = -INFINITY, tile_b = -INFINITY;
        const int warp_first = first_pos + r0, warp_last = warp_first + 15;
        const bool open = r0 + 15 < n_rows && kt + kKeys - 1 <= warp_first && kt >= first_visible(warp_last, s);
        if (open && plain_scores) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                S[nt][0] *= s.scale; S[nt][1] *= s.scale; S[nt][2] *= s.scale; S[nt][3] *= s.scale;
                tile_a = fmaxf(tile_a, fmaxf(S[nt][0], S[nt][1]));
                tile_b = fmaxf(tile_b, fmaxf(S[nt][2], S[nt][3]));
            }
        } else {
            // key - position of this thread's first key of the tile, for its two rows; the other keys lie a constant further.
            const float back_a = static_cast<float>(kt + 2 * t - pos_a), back_b = static_cast<float>(kt + 2 * t - pos_b);
            auto shape = [&](auto capped_tag, auto masked_tag) {
                constexpr bool kCapped = decltype(capped_tag)::value, kMasked = decltype(masked_tag)::value;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const bool upper = e < 2;
                        const float further = static_cast<float>(nt * 8 + (e & 1));
                        float v = tile_score<kCapped>(S[nt][e], (upper ? back_a : back_b) + further, to_cap, s.softcap, slope);
                        if (kMasked) {
                            const int key = kt + nt * 8 + 2 * t + (e & 1);
                            const bool seen = upper ? (row_a && key <= pos_a && (key >= lo_a || key < keep_first))
                                                    : (row_b && key <= pos_b && (key >= lo_b || key < keep_first));
                            if (!seen) v = -INFINITY;
                        }
                        S[nt][e] = v;
                        if (upper) tile_a = fmaxf(tile_a, v); else tile_b = fmaxf(tile_b, v);
                    }
            };
            if (open) {
                if (capped) shape(std::true_type{}, std::false_type{});
                else shape(std::false_type{}, std::false_type{});
            } else {
                if (capped) shape(std::true_type{}, std::true_type{});
                else shape(std::false_type{}, std::true_type{});
            }
        }
        tile_a = fmaxf(tile_a, __shfl_xor_sync(0xffffffffu, tile_a, 1));
        tile_a = fmaxf(tile_a, __shfl_xor_sync(0xffffffffu, tile_a, 2));
        tile_b = fmaxf(tile_b, __shfl_xor_sync(0xffffffffu, tile_b, 1));
        tile_b = fmaxf(tile_b, __shfl_xor_sync(0xffffffffu, tile_b, 2));
        const float new_a = fmaxf(m_a, tile_a), new_b = fmaxf(m_b, tile_b);
        const float alpha_a = (m_a == -INFINITY) ? 0.0f : __expf(m_a - new_a);
        const float alpha_b = (m_b == -INFINITY) ? 0.0f : __expf(m_b - new_b);
        m_a = new_a;
        m_b = new_b;
        l_a *= alpha_a;
        l_b *= alpha_b;
#pragma unroll
        for (int nv = 0; nv < NV; ++nv) {
            O[nv][0] *= alpha_a; O[nv][1] *= alpha_a; O[nv][2] *= alpha_b; O[nv][3] *= alpha_b;
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float m = e < 2 ? new_a : new_b;
                const float p = S[nt][e] == -INFINITY ? 0.0f : __expf(S[nt][e] - m);     // ex2.approx: 2 ulp, weights stay float32
                S[nt][e] = p;
                if (e < 2) l_a += p; else l_b += p;
            }
        // O += P V, P as hi + lo
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p0 = S[2 * kk + (j >> 1)][(j & 1) * 2], p1 = S[2 * kk + (j >> 1)][(j & 1) * 2 + 1];
                const __nv_bfloat16 h0 = __float2bfloat16_rn(p0), h1 = __float2bfloat16_rn(p1);
                hi[j] = pack_bf16(__bfloat162float(h0), __bfloat162float(h1));
                lo[j] = pack_bf16(p0 - __bfloat162float(h0), p1 - __bfloat162float(h1));
            }
            const uint32_t row_addr = vt_base + static_cast<uint32_t>(((kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vstride + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int nv = 0; nv < NV; nv += 2) {
                if (nv * 8 < s.vdim) {          // the second tile of a pair may lie in the row's padding: it is computed and never stored
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, row_addr + nv * 16);
                    mma_bf16(O[nv], hi, vb[0], vb[1]);
                    mma_bf16(O[nv], lo, vb[0], vb[1]);
                    mma_bf16(O[nv + 1], hi, vb[2], vb[3]);
                    mma_bf16(O[nv + 1], lo, vb[2], vb[3]);
                }
            }
        }
    }
    mlr_grid_dependents_may_start();     // only now: blocks of the next grid that wait on this SM would take its room
    if (bad && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) {
        if (nv * 8 >= s.vdim) continue;
        const int col = head * s.vdim + nv * 8 + 2 * t;
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            if (!(hb ? row_b : row_a)) continue;
            const float l = hb ? l_b : l_a;
            float v0 = l > 0.0f ? O[nv][2 * hb] / l : 0.0f, v1 = l > 0.0f ? O[nv][2 * hb + 1] / l : 0.0f;
            const size_t row = static_cast<size_t>(first + tile_token + r0 + g + 8 * hb);
            if (gate && s.gate_kind == 3) {
                const float one = mlr_gate_value(__bfloat162float(gate[row * ld_gate + head]), 3);
                v0 *= one;
                v1 *= one;
            } else if (gate) {
                v0 *= mlr_gate_value(__bfloat162float(gate[row * ld_gate + col]), s.gate_kind);
                v1 *= mlr_gate_value(__bfloat162float(gate[row * ld_gate + col + 1]), s.gate_kind);
            }
            *reinterpret_cast<__nv_bfloat162*>(out + row * ldo + col) = __floats2bfloat162_rn(v0 * s.out_scale, v1 * s.out_scale);
        }
    }
}

// ---- few rows per request in bfloat16 (decoded tokens, short portions): one block per (segment, kv head, range of keys) takes
// ALL query heads that share the kv head, so the keys and values of a range are read once for the group.  The heads of the
// group are the rows of the tensor-core tiles (up to 16; rows past the group are zeros): S = Q K^T by mma.sync, mask and
// softmax in float32, the weights as two bfloat16 terms against the values, float32 sums, as in the tile kernel above.  A
// tile of 64 keys is cut over the four warps (16 keys each, every warp with a running maximum and sums of its own); at the
// end the warps' results are added up in shared memory and go to `partial` in the row kernel's layout (the same merge
// kernel follows), or, when the block has seen every key of the row, straight to the output.
template <int NV>
__global__ void __launch_bounds__(128, NV >= 16 ? 3 : 4) attention_masked_group_kernel(const __nv_bfloat16* q, int ldq, const __nv_bfloat16* gate, int ld_gate,
                                                                     __nv_bfloat16* out, int ldo, const __nv_bfloat16* cache, int num_pages,
                                                                     const int* positions, const int* segment_of_row, const int* block_table,
                                                                     int table_stride, int page_size, MaskedAttentionSpec s, const int* items,
                                                                     const int* segment_info, int split_keys, int max_splits, float* partial,
                                                                     int* status) {
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int qstride = s.dim + kPad, vstride = s.shared_kv ? qstride : s.vdim + kPad;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* Ks = Qs + 16 * qstride;
    __nv_bfloat16* Vs = s.shared_kv ? Ks : Ks + 2 * kKeys * qstride;        // two stages of each; values that are their keys' start are read there
    float* merged = reinterpret_cast<float*>(Ks);                            // [4 warps][16 rows][vdim + 2], once the last tile is done
    __shared__ int bad;

    const int* info = segment_info + 4 * (items ? items[blockIdx.x] : blockIdx.x);
    const int first_row = info[0], n_rows = min(info[1], kRowsPerItem);
    // More than 16 heads on a kv head: blocks of their own take them 16 at a time (`group`: this block's heads).
    const int sharing = s.heads / s.kv_heads, chunks = (sharing + 15) / 16;
    const int kv_head = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
    const int head0 = kv_head * sharing + chunk * 16, group = min(16, sharing - chunk * 16);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const size_t page_elems = static_cast<size_t>(s.kv_heads) * page_size * (s.shared_kv ? s.dim : s.dim + s.vdim);
    const size_t key_plane = s.shared_kv ? 0 : static_cast<size_t>(s.kv_heads) * page_size * s.dim;
    const bool capped = s.softcap > 0.0f;
    const float to_cap = capped ? 2.0f * 1.4426950408889634f * s.scale / s.softcap : s.scale;
    const float slope_a = (s.slopes && g < group) ? s.slopes[head0 + g] : 0.0f;
    const float slope_b = (s.slopes && g + 8 < group) ? s.slopes[head0 + g + 8] : 0.0f;
    const int ksteps = s.dim / 16, half = s.rot_dims / 2, mstride = s.vdim + 2;
    const uint32_t qs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Qs));
    const uint32_t ks_base = static_cast<uint32_t>(__cvta_generic_to_shared(Ks));
    const uint32_t vs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vs));
    if (threadIdx.x == 0) bad = 0;

    for (int j = 0; j < n_rows; ++j) {
        __syncthreads();            // the row before is done with the shared memory
        const int row = first_row + j;
        const int position = positions[row];
        const int* table = block_table + static_cast<size_t>(segment_of_row[row]) * table_stride;
        const int lo = first_visible(position, s);
        const int kept = (s.window > 0 && s.keep_first > 0) ? min(s.keep_first, lo) : 0;       // keys [0, kept) are seen beside [lo, position]
        int tile_first = (lo / kKeys) * kKeys, tile_last = position;
        if (partial) {
            tile_first += blockIdx.z * split_keys;
            tile_last = min(position, tile_first + split_keys - 1);
            if (tile_first > position) continue;           // the merge reads only the ranges that exist for this row
        }
        const int kept_tiles = (kept > 0 && (!partial || blockIdx.z == 0)) ? (kept + kKeys - 1) / kKeys : 0;
        const int all_tiles = kept_tiles + (tile_last - tile_first) / kKeys + 1;
        auto tile_start = [&](int i) { return i < kept_tiles ? i * kKeys : tile_first + (i - kept_tiles) * kKeys; };
        // Keys (and values) of a tile go into one of two stages by asynchronous copies, two threads per key; keys the row does
        // not see become zeros.
        auto page_for = [&](int i) {      // read one tile before `fetch` needs it; 0 for a key the row does not see
            const bool early = i < kept_tiles;
            const int at = tile_start(i) + (threadIdx.x >> 1);
            return (at >= (early ? 0 : lo) && at <= (early ? kept - 1 : tile_last)) ? __ldg(table + at / page_size) : 0;
        };
        auto fetch = [&](int i, int into, int page) {
            const bool early = i < kept_tiles;
            const int see_lo = early ? 0 : lo, see_hi = early ? kept - 1 : tile_last;
            const int key = threadIdx.x >> 1, at = tile_start(i) + key;
            bool real = at >= see_lo && at <= see_hi;
            const __nv_bfloat16* ksrc = cache;
            const __nv_bfloat16* vsrc = cache;
            if (real) {
                if (page < 0 || page >= num_pages) {
                    bad = 1;
                    real = false;
                } else {
                    const size_t in_page = static_cast<size_t>(kv_head) * page_size + at % page_size;
                    ksrc = cache + page * page_elems + in_page * s.dim;
                    vsrc = cache + page * page_elems + key_plane + in_page * s.vdim;
                }
            }
            __nv_bfloat16* krow = Ks + (into * kKeys + key) * qstride;
            for (int c = (threadIdx.x & 1) * 8; c < s.dim; c += 16) mlr_async_copy16(krow + c, real ? ksrc + c : cache, real);
            if (!s.shared_kv) {
                __nv_bfloat16* vrow = Vs + (into * kKeys + key) * vstride;
                for (int c = (threadIdx.x & 1) * 8; c < s.vdim; c += 16) mlr_async_copy16(vrow + c, real ? vsrc + c : cache, real);
            }
            mlr_async_commit();
        };
        // The first tile's copies are on their way while the queries are made ready.
        fetch(0, 0, page_for(0));
        int page_ahead = all_tiles > 1 ? page_for(1) : 0;
        // The group's queries, rotated in float32, as bfloat16.
        for (int i = threadIdx.x; i < 16 * s.dim; i += 128) {
            const int r = i / s.dim, c = i % s.dim;
            float value = 0.0f;
            if (r < group) {
                const __nv_bfloat16* qrow = q + static_cast<size_t>(row) * ldq + static_cast<size_t>(head0 + r) * s.dim;
                value = __bfloat162float(qrow[c]);
                if (c < s.rot_dims) {
                    float sn, cs;
                    sincosf(static_cast<float>(position) * s.freq[c < half ? c : c - half], &sn, &cs);
                    const float other = __bfloat162float(qrow[c < half ? c + half : c - half]);
                    value = c < half ? value * cs - other * sn : value * cs + other * sn;
                }
            }
            Qs[r * qstride + c] = __float2bfloat16_rn(value);
        }
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
        float O[NV][4];
#pragma unroll
        for (int nv = 0; nv < NV; ++nv) O[nv][0] = O[nv][1] = O[nv][2] = O[nv][3] = 0.0f;
        int current = 0;
        for (int ti = 0; ti < all_tiles; ++ti, current ^= 1) {
            const bool early = ti < kept_tiles;
            const int kt = tile_start(ti), see_lo = early ? 0 : lo, see_hi = early ? kept - 1 : tile_last;
            mlr_async_wait();
            __syncthreads();      // this tile has arrived (and Qs is written); no warp still reads the other stage
            if (ti + 1 < all_tiles) {
                fetch(ti + 1, current ^ 1, page_ahead);
                if (ti + 2 < all_tiles) page_ahead = page_for(ti + 2);
            }
            const uint32_t kt_base = ks_base + static_cast<uint32_t>(current * kKeys * qstride * 2);
            const uint32_t vt_base = vs_base + static_cast<uint32_t>(current * kKeys * vstride * 2);
            float S[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.0f;
            const uint32_t q_row = qs_base + static_cast<uint32_t>((((lane & 7) + ((lane >> 3) & 1) * 8) * qstride + (lane >> 4) * 8) * 2);
            const uint32_t k_row = kt_base + static_cast<uint32_t>(((warp * 16 + (lane & 7)) * qstride + (lane >> 3) * 8) * 2);
            for (int ks = 0; ks < ksteps; ks += 2) {
                uint32_t a[4], a2[4] = {0, 0, 0, 0};
                ldmatrix_x4(a, q_row + ks * 32);
                const bool two = ks + 1 < ksteps;
                if (two) ldmatrix_x4(a2, q_row + (ks + 1) * 32);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    uint32_t kb[4];
                    const uint32_t at = k_row + static_cast<uint32_t>((nt * 8 * qstride + ks * 16) * 2);
                    if (two) {
                        ldmatrix_x4(kb, at);
                        mma_bf16(S[nt], a, kb[0], kb[1]);
                        mma_bf16(S[nt], a2, kb[2], kb[3]);
                    } else {
                        ldmatrix_x2(kb, at);
                        mma_bf16(S[nt], a, kb[0], kb[1]);
                    }
                }
            }
            // All rows of the block are heads at ONE position: a key is seen by all of them or by none.
            const int key0 = kt + warp * 16 + 2 * t;
            const float back = static_cast<float>(key0 - position);
            float tile_a = -INFINITY, tile_b = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + nt * 8 + (e & 1);
                    const float further = static_cast<float>(nt * 8 + (e & 1));
                    float v = capped ? tile_score<true>(S[nt][e], back + further, to_cap, s.softcap, e < 2 ? slope_a : slope_b)
                                     : tile_score<false>(S[nt][e], back + further, to_cap, 0.0f, e < 2 ? slope_a : slope_b);
                    if (key < see_lo || key > see_hi) v = -INFINITY;
                    S[nt][e] = v;
                    if (e < 2) tile_a = fmaxf(tile_a, v); else tile_b = fmaxf(tile_b, v);
                }
            tile_a = fmaxf(tile_a, __shfl_xor_sync(0xffffffffu, tile_a, 1));
            tile_a = fmaxf(tile_a, __shfl_xor_sync(0xffffffffu, tile_a, 2));
            tile_b = fmaxf(tile_b, __shfl_xor_sync(0xffffffffu, tile_b, 1));
            tile_b = fmaxf(tile_b, __shfl_xor_sync(0xffffffffu, tile_b, 2));
            const float new_a = fmaxf(m_a, tile_a), new_b = fmaxf(m_b, tile_b);
            const float alpha_a = (m_a == -INFINITY) ? 0.0f : __expf(m_a - new_a);
            const float alpha_b = (m_b == -INFINITY) ? 0.0f : __expf(m_b - new_b);
            m_a = new_a;
            m_b = new_b;
            l_a *= alpha_a;
            l_b *= alpha_b;
#pragma unroll
            for (int nv = 0; nv < NV; ++nv) {
                O[nv][0] *= alpha_a; O[nv][1] *= alpha_a; O[nv][2] *= alpha_b; O[nv][3] *= alpha_b;
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float m = e < 2 ? new_a : new_b;
                    const float p = S[nt][e] == -INFINITY ? 0.0f : __expf(S[nt][e] - m);
                    S[nt][e] = p;
                    if (e < 2) l_a += p; else l_b += p;
                }
            // O += P V over the warp's 16 keys, P as hi + lo
            uint32_t hi[4], lo2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p0 = S[i >> 1][(i & 1) * 2], p1 = S[i >> 1][(i & 1) * 2 + 1];
                const __nv_bfloat16 h0 = __float2bfloat16_rn(p0), h1 = __float2bfloat16_rn(p1);
                hi[i] = pack_bf16(__bfloat162float(h0), __bfloat162float(h1));
                lo2[i] = pack_bf16(p0 - __bfloat162float(h0), p1 - __bfloat162float(h1));
            }
            const uint32_t row_addr = vt_base + static_cast<uint32_t>(((warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vstride + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int nv = 0; nv < NV; nv += 2) {
                if (nv * 8 < s.vdim) {          // the second tile of a pair may lie in the row's padding: it is computed and never stored
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, row_addr + nv * 16);
                    mma_bf16(O[nv], hi, vb[0], vb[1]);
                    mma_bf16(O[nv], lo2, vb[0], vb[1]);
                    mma_bf16(O[nv + 1], hi, vb[2], vb[3]);
                    mma_bf16(O[nv + 1], lo2, vb[2], vb[3]);
                }
            }
        }
        // The four warps' maxima, sums and weighted values side by side in shared memory, then added up head by head.
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        __syncthreads();          // every warp is done with the tiles: their room becomes `merged`
        {
            float* mine_a = merged + (warp * 16 + g) * mstride;
            float* mine_b = merged + (warp * 16 + g + 8) * mstride;
            if (t == 0) {
                mine_a[0] = m_a; mine_a[1] = l_a;
                mine_b[0] = m_b; mine_b[1] = l_b;
            }
#pragma unroll
            for (int nv = 0; nv < NV; ++nv) {
                const int c = nv * 8 + 2 * t;
                if (c < s.vdim) {
                    mine_a[2 + c] = O[nv][0]; mine_a[2 + c + 1] = O[nv][1];
                    mine_b[2 + c] = O[nv][2]; mine_b[2 + c + 1] = O[nv][3];
                }
            }
        }
        __syncthreads();
        for (int r = 0; r < group; ++r) {
            const int head = head0 + r;
            float top = -INFINITY, w[4], sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) top = fmaxf(top, merged[(i * 16 + r) * mstride]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float m = merged[(i * 16 + r) * mstride];
                w[i] = m == -INFINITY ? 0.0f : expf(m - top);
                sum = fmaf(merged[(i * 16 + r) * mstride + 1], w[i], sum);
            }
            if (partial) {
                float* mine = partial + ((static_cast<size_t>(blockIdx.x) * partial_slots(s) + j * s.heads + head) * max_splits +
                                         blockIdx.z) * mstride;
                if (threadIdx.x == 0) {
                    mine[0] = top;
                    mine[1] = sum;
                }
                for (int c = threadIdx.x; c < s.vdim; c += 128) {
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc = fmaf(merged[(i * 16 + r) * mstride + 2 + c], w[i], acc);
                    mine[2 + c] = acc;
                }
            } else {
                // The block saw every key of the row: the sink joins here, and the row is finished.
                float scale_all = 1.0f;
                if (s.sink) {
                    const float sink_score = s.sinks ? s.sinks[head] : 0.0f;
                    const float both = fmaxf(top, sink_score);
                    scale_all = top == -INFINITY ? 0.0f : expf(top - both);
                    sum = fmaf(sum, scale_all, expf(sink_score - both));
                }
                __nv_bfloat16* orow = out + static_cast<size_t>(row) * ldo + static_cast<size_t>(head) * s.vdim;
                const __nv_bfloat16* grow = gate ? gate + static_cast<size_t>(row) * ld_gate + static_cast<size_t>(head) * (s.gate_kind == 3 ? 1 : s.vdim) : nullptr;
                for (int c = threadIdx.x; c < s.vdim; c += 128) {
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc = fmaf(merged[(i * 16 + r) * mstride + 2 + c], w[i], acc);
                    float value = sum > 0.0f ? acc * scale_all / sum : 0.0f;
                    if (grow) value *= mlr_gate_value(__bfloat162float(grow[s.gate_kind == 3 ? 0 : c]), s.gate_kind);
                    orow[c] = __float2bfloat16_rn(value * s.out_scale);
                }
            }
        }
    }
    if (bad && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
    mlr_grid_dependents_may_start();
}

int check_spec(const MaskedAttentionSpec* s, const char* who) {
    MLR_REQUIRE(s, "%s: no description", who);
    MLR_REQUIRE(s->heads > 0 && s->kv_heads > 0 && s->heads % s->kv_heads == 0, "%s: %d query heads cannot share %d kv heads", who,
                s->heads, s->kv_heads);
    MLR_REQUIRE(s->dim >= 1 && s->dim <= 1024 && s->vdim >= 1 && s->vdim <= kThreads * kMaxDimsPerThread,
                "%s: key size %d or value size %d is outside what the kernel takes (1024, %d)", who, s->dim, s->vdim,
                kThreads * kMaxDimsPerThread);
    MLR_REQUIRE(s->rot_dims >= 0 && s->rot_dims % 2 == 0 && s->rot_dims <= s->dim && (s->rot_dims == 0 || s->freq),
                "%s: %d rotated values do not fit a head of %d (or no frequencies were given)", who, s->rot_dims, s->dim);
    MLR_REQUIRE(s->window >= 0 && s->chunk >= 0 && s->heads <= 65535, "%s: bad window, chunk or head count", who);
    MLR_REQUIRE(!s->shared_kv || s->vdim <= s->dim, "%s: values that are the start of their keys cannot be longer, %d against %d", who, s->vdim, s->dim);
    MLR_REQUIRE(s->keep_first >= 0 && (s->keep_first == 0 || (s->window > 0 && s->chunk == 0)), "%s: kept first tokens go with a window and without chunks", who);
    MLR_REQUIRE(s->gate_kind >= 0 && s->gate_kind <= 3 && (!s->sinks || s->sink), "%s: bad gate kind, or sink scores without a sink", who);
    MLR_REQUIRE(!s->dense_cache || (s->dim == s->vdim && !s->shared_kv), "%s: the plain attention kernels' cache has keys and values of one size", who);
    return 0;
}

}  // namespace

MLR_API int mlr_kv_rope_cache(const MaskedAttentionSpec* spec, const void* k, int ld_k, const void* v, int ld_v, int act_bf16,
                              void* cache, int num_pages, const int* positions, const int* segment_of_row, const int* block_table,
                              int table_stride, int page_size, int rows, int* status, cudaStream_t stream) {
    if (check_spec(spec, "kv_rope_cache")) return 1;
    MLR_REQUIRE(rows >= 0 && page_size > 0 && num_pages > 0 && cache && block_table, "kv_rope_cache: bad sizes or no cache");
    MLR_REQUIRE(ld_k >= spec->kv_heads * spec->dim && ld_v >= spec->kv_heads * spec->vdim, "kv_rope_cache: a row stride is smaller than the row");
    if (rows == 0) return 0;
    if (act_bf16)
        mlr_launch((kv_rope_cache_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const __nv_bfloat16*>(k), ld_k,
                   static_cast<const __nv_bfloat16*>(v), ld_v, static_cast<__nv_bfloat16*>(cache), num_pages, positions, segment_of_row,
                   block_table, table_stride, page_size, *spec, status);
    else
        mlr_launch((kv_rope_cache_kernel<float>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const float*>(k), ld_k,
                   static_cast<const float*>(v), ld_v, static_cast<float*>(cache), num_pages, positions, segment_of_row, block_table,
                   table_stride, page_size, *spec, status);
    return mlr_launched("kv_rope_cache");
}

// q, k, v: the step's projections (q is changed in place); bq, bk, bv: float32 biases or null; first: float32 [rows, kv_heads * vdim]
// (row stride ld_first) with mix 1 (written) or 2 (read), else null.  Not for caches whose values are their keys.
// The description's qk_norm, q_weight and k_weight name a weighted norm of q and k.  With k, v and cache null the layer reads another layer's cache and only its queries are prepared.
MLR_API int mlr_qkv_prepare_cache(const MaskedAttentionSpec* spec, void* q, int ldq, const void* k, int ld_k, const void* v, int ld_v, int act_bf16,
                                  const float* bq, const float* bk, const float* bv, int unit_qk, int unit_v, float eps, float* first, int ld_first,
                                  int mix, float lambda, void* cache, int num_pages, const int* positions, const int* segment_of_row,
                                  const int* block_table, int table_stride, int page_size, int rows, int* status, cudaStream_t stream) {
    if (check_spec(spec, "qkv_prepare_cache")) return 1;
    const bool own_kv = k != nullptr;
    const float* wq = spec->q_weight;
    const float* wk = spec->k_weight;
    const int qk_norm = spec->qk_norm;
    MLR_REQUIRE(rows >= 0 && page_size > 0 && q, "qkv_prepare_cache: bad sizes or no queries");
    MLR_REQUIRE(own_kv ? (v && cache && block_table && num_pages > 0) : (!v && !cache && mix == 0),
                "qkv_prepare_cache: keys, values and the cache come together or not at all");
    MLR_REQUIRE(!spec->shared_kv, "qkv_prepare_cache: this cache keeps keys and values apart");
    MLR_REQUIRE(ldq >= spec->heads * spec->dim && (!own_kv || (ld_k >= spec->kv_heads * spec->dim && ld_v >= spec->kv_heads * spec->vdim)),
                "qkv_prepare_cache: a row stride is smaller than the row");
    MLR_REQUIRE(mix >= 0 && mix <= 2 && (mix == 0 || (first && ld_first >= spec->kv_heads * spec->vdim)), "qkv_prepare_cache: mixing needs the first values' buffer");
    MLR_REQUIRE(qk_norm >= 0 && qk_norm <= 2 && (qk_norm == 0 || (wq && (wk || !own_kv) && eps > 0.0f)),
                "qkv_prepare_cache: a weighted norm of q and k needs its weights and a positive eps");
    if (rows == 0) return 0;
    // A norm over the whole projection reads all of q before any of it is changed: one block a row; with few rows that block gets a
    // warp per head (up to 32), so that the heads' loads are in flight together.
    const int all_units = own_kv ? spec->heads + 2 * spec->kv_heads : spec->heads;
    int threads = kThreads;
    if (qk_norm == 2 && rows <= 64) threads = 32 * (all_units < 32 ? (all_units < 4 ? 4 : all_units) : 32);
    const size_t shared = sizeof(float) * (threads / 32) * static_cast<size_t>(spec->dim > spec->vdim ? spec->dim : spec->vdim);
    MLR_REQUIRE(shared <= 160 * 1024, "qkv_prepare_cache: heads of %d values do not fit shared memory", spec->dim > spec->vdim ? spec->dim : spec->vdim);
    // With few rows (decoded tokens) every warp takes one head of q, k or v; with many, a block of four warps walks its row's
    // heads in turn, which the same number of blocks in flight does a little faster.
    const int units = all_units, warps = threads / 32;
    const int wanted = rows >= 592 || qk_norm == 2 ? 1 : (592 + rows - 1) / rows, most = (units + warps - 1) / warps;
    const dim3 grid(rows, wanted < most ? wanted : most);
#define MLR_PREPARE(T, BLOCK)                                                                                                              \
    do {                                                                                                                                   \
        if (shared > 48 * 1024)                                                                                                            \
            cudaFuncSetAttribute(qkv_prepare_cache_kernel<T, BLOCK>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)); \
        mlr_launch((qkv_prepare_cache_kernel<T, BLOCK>), dim3(grid), dim3(threads), shared, stream, static_cast<T*>(q), ldq,               \
                   static_cast<const T*>(k), ld_k, static_cast<const T*>(v), ld_v, bq, bk, bv, unit_qk, unit_v, eps, first, ld_first, mix, \
                   lambda, static_cast<T*>(cache), num_pages, positions, segment_of_row, block_table, table_stride, page_size, *spec,      \
                   status);                                                                                                                \
    } while (0)
    if (act_bf16) {
        if (threads == kThreads) MLR_PREPARE(__nv_bfloat16, kThreads);
        else MLR_PREPARE(__nv_bfloat16, kPrepareThreads);
    } else {
        if (threads == kThreads) MLR_PREPARE(float, kThreads);
        else MLR_PREPARE(float, kPrepareThreads);
    }
#undef MLR_PREPARE
    return mlr_launched("qkv_prepare_cache");
}

MLR_API int mlr_attention_masked(const MaskedAttentionSpec* spec, const void* q, int ldq, const void* gate, int ld_gate, void* out,
                                 int ldo, int act_bf16, const void* cache, int num_pages, const int* positions,
                                 const int* segment_of_row, const int* block_table, int table_stride, int page_size, int rows,
                                 const int* items, int n_items, const int* segment_info, int split_keys, int max_splits,
                                 int finer, float* partial, int* status, cudaStream_t stream) {
    // With `segment_info` the kernel runs over `n_items` segments of at most 16 rows each (`items` lists them; null: the
    // step's first n_items segments) and `rows` is not used; without it, over all `rows` rows.  With `partial` (float32,
    // n_items * max(16 * kv_heads, heads rounded up to 16) * max_splits * (vdim + 2); segments of at most 16 / (heads / kv_heads)
    // rows, of one row where more than 16 heads share a kv head) and more than one split, every row's keys are cut into ranges of `split_keys` that run as blocks of their own, and a second
    // kernel adds the ranges up.
    if (check_spec(spec, "attention_masked")) return 1;
    if (segment_info) rows = n_items;          // a block per segment; it walks the segment's rows
    if (!partial || max_splits <= 1 || !segment_info) {
        partial = nullptr;
        max_splits = 1;
    } else {
        MLR_REQUIRE(split_keys >= kTile && split_keys % kTile == 0 && max_splits <= 65535 && finer >= 1, "attention_masked: bad key split %d x %d",
                    split_keys, max_splits);
        // `finer`: the caller's `partial` has room for that many times `max_splits` ranges; each planned range is cut
        // further (down to two tiles of keys) so that more blocks have loads in flight at once.
        if (finer > 1) {
            const long long span = static_cast<long long>(split_keys) * max_splits;
            const int tiles = split_keys / kTile;
            const int fewer = tiles / finer >= 2 ? (tiles + finer - 1) / finer : (tiles >= 2 ? 2 : tiles);    // tiles of a finer range
            const long long ranges = (span + static_cast<long long>(fewer) * kTile - 1) / (static_cast<long long>(fewer) * kTile);
            if (ranges <= static_cast<long long>(max_splits) * finer && ranges <= 65535) {
                split_keys = fewer * kTile;
                max_splits = static_cast<int>(ranges);
            }
        }
    }
    MLR_REQUIRE(rows >= 0 && page_size > 0 && num_pages > 0, "attention_masked: bad page size or page count");
    MLR_REQUIRE(ldq >= spec->heads * spec->dim && ldo >= spec->heads * spec->vdim, "attention_masked: a row stride is smaller than the row");
    MLR_REQUIRE((spec->gate_kind == 0) == (gate == nullptr), "attention_masked: the description and the call disagree about a gate");
    if (rows == 0) return 0;
    const size_t shared = sizeof(float) * (spec->dim + kTile) + sizeof(long long) * kTile + 16;
    const dim3 grid(rows, spec->heads, max_splits);
    const dim3 merge_grid(rows, spec->heads);
    const int group = spec->heads / spec->kv_heads;
    if (act_bf16 && segment_info && spec->dim % 16 == 0 && spec->dim <= 256 && spec->vdim % 8 == 0 && spec->vdim <= 128 &&
        reinterpret_cast<uintptr_t>(cache) % 16 == 0) {
        // Few rows per request in bfloat16: the query heads of a kv head share one block (and one reading of the keys).
        const size_t stages = sizeof(__nv_bfloat16) * (static_cast<size_t>(16 + 2 * kKeys) * (spec->dim + kPad) +
                                                       (spec->shared_kv ? 0 : 2 * kKeys * (spec->vdim + kPad)));
        const size_t sums = sizeof(__nv_bfloat16) * 16 * (spec->dim + kPad) + sizeof(float) * 4 * 16 * (spec->vdim + 2);
        const size_t group_shared = stages > sums ? stages : sums;
        const dim3 group_grid(rows, spec->kv_heads * ((group + 15) / 16), max_splits);     // more than 16 heads on a kv head: 16 a block
#define MLR_GROUP(NV)                                                                                                                       \
    do {                                                                                                                                    \
        cudaFuncSetAttribute(attention_masked_group_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(group_shared)); \
        mlr_launch((attention_masked_group_kernel<NV>), dim3(group_grid), dim3(128), group_shared, stream,                                  \
                   static_cast<const __nv_bfloat16*>(q), ldq, static_cast<const __nv_bfloat16*>(gate), ld_gate,                              \
                   static_cast<__nv_bfloat16*>(out), ldo, static_cast<const __nv_bfloat16*>(cache), num_pages, positions, segment_of_row,    \
                   block_table, table_stride, page_size, *spec, items, segment_info, split_keys, max_splits, partial, status);              \
    } while (0)
        if (spec->vdim <= 32) MLR_GROUP(4);
        else if (spec->vdim <= 64) MLR_GROUP(8);
        else if (spec->vdim <= 96) MLR_GROUP(12);
        else MLR_GROUP(16);
#undef MLR_GROUP
        if (partial)
            mlr_launch((attention_masked_merge_kernel<__nv_bfloat16, 2>), dim3(merge_grid), dim3(kThreads), 0, stream, partial,
                       static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__nv_bfloat16*>(out), ldo, positions, *spec, items,
                       segment_info, split_keys, max_splits);
        return mlr_launched("attention_masked");
    }
#define MLR_ROWS(T, DPT)                                                                                                                    \
    do {                                                                                                                                    \
        mlr_launch((attention_masked_kernel<T, DPT>), dim3(grid), dim3(kThreads), shared, stream, static_cast<const T*>(q), ldq,            \
                   static_cast<const T*>(gate), ld_gate, static_cast<T*>(out), ldo, static_cast<const T*>(cache), num_pages, positions,     \
                   segment_of_row, block_table, table_stride, page_size, *spec, items, segment_info, split_keys, max_splits, partial,       \
                   status);                                                                                                                 \
        if (partial)                                                                                                                        \
            mlr_launch((attention_masked_merge_kernel<T, DPT>), dim3(merge_grid), dim3(kThreads), 0, stream, partial,                       \
                       static_cast<const T*>(gate), ld_gate, static_cast<T*>(out), ldo, positions, *spec, items, segment_info, split_keys,  \
                       max_splits);                                                                                                         \
    } while (0)
#define MLR_COLUMNS(T)                                          \
    do {                                                        \
        if (spec->vdim <= 2 * kThreads) MLR_ROWS(T, 2);         \
        else if (spec->vdim <= 4 * kThreads) MLR_ROWS(T, 4);    \
        else MLR_ROWS(T, 8);                                    \
    } while (0)
    if (act_bf16) MLR_COLUMNS(__nv_bfloat16);
    else MLR_COLUMNS(float);
#undef MLR_COLUMNS
#undef MLR_ROWS
    return mlr_launched("attention_masked");
}

// Whether the tiled kernel takes these sizes (bfloat16 only): 1 yes, 0 no.
MLR_API int mlr_attention_masked_tiles_fit(int dim, int vdim) {
    return dim % 16 == 0 && dim >= 16 && dim <= 256 && vdim % 8 == 0 && vdim >= 8 && vdim <= 128;
}

// tiles: n_tiles pairs {segment, first token of a tile of up to 64 rows of that segment}.
MLR_API int mlr_attention_masked_tiles(const MaskedAttentionSpec* spec, const void* q, int ldq, const void* gate, int ld_gate, void* out,
                                       int ldo, const void* cache, int num_pages, const int* tiles, int n_tiles,
                                       const int* segment_info, const int* block_table, int table_stride, int page_size, int* status,
                                       cudaStream_t stream) {
    if (check_spec(spec, "attention_masked_tiles")) return 1;
    MLR_REQUIRE(mlr_attention_masked_tiles_fit(spec->dim, spec->vdim), "attention_masked_tiles: key size %d / value size %d not taken",
                spec->dim, spec->vdim);
    MLR_REQUIRE(n_tiles >= 0 && n_tiles <= 65535 && page_size > 0 && num_pages > 0, "attention_masked_tiles: bad tile count or pages");
    MLR_REQUIRE(ldq >= spec->heads * spec->dim && ldo >= spec->heads * spec->vdim && ldo % 2 == 0 && (spec->heads * spec->vdim) % 2 == 0,
                "attention_masked_tiles: bad row strides");
    MLR_REQUIRE((spec->gate_kind == 0) == (gate == nullptr), "attention_masked_tiles: the description and the call disagree about a gate");
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(cache) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0, "attention_masked_tiles: alignment");
    if (n_tiles == 0) return 0;
    const size_t shared = sizeof(__nv_bfloat16) * (static_cast<size_t>(kRows + 2 * kKeys) * (spec->dim + kPad) +
                                                   (spec->shared_kv ? 0 : 2 * kKeys * (spec->vdim + kPad)));
    const dim3 grid(spec->heads, n_tiles);
#define MLR_TILES(NV)                                                                                                              \
    do {                                                                                                                           \
        cudaFuncSetAttribute(attention_masked_tile_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)); \
        mlr_launch((attention_masked_tile_kernel<NV>), dim3(grid), dim3(128), shared, stream, static_cast<const __nv_bfloat16*>(q), ldq, \
                   static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__nv_bfloat16*>(out), ldo,                         \
                   static_cast<const __nv_bfloat16*>(cache), num_pages, tiles, segment_info, block_table, table_stride, page_size, \
                   *spec, status);                                                                                                 \
    } while (0)
    if (spec->vdim <= 32) MLR_TILES(4);
    else if (spec->vdim <= 64) MLR_TILES(8);
    else if (spec->vdim <= 96) MLR_TILES(12);
    else MLR_TILES(16);
#undef MLR_TILES
    return mlr_launched("attention_masked_tiles");
}
