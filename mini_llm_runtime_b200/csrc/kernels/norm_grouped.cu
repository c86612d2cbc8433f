// RMS norm in groups, on the float32 residual stream, as the two halves of a block that norms
// both what goes into a sub-layer and what comes out of it:
//
//   if delta:  h[row] += groupnorm(delta[row] + bias) * w_post      (the sub-layer's result, normed, joins the stream;
//                                                                   with norm_delta = 0 it joins as it is)
//   if out:    out[r]  = groupnorm(h[row]) * w_pre                  (the next sub-layer's input; with bit 1 of `norm_delta`
//                                                                   set it is h[row] itself: a sub-layer without a norm in front)
//
// groupnorm(x): x in `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps).
// groups = 1 is the ordinary RMS norm.  row = rows[r] when an index list is given (the wanted rows
// before the head), else r.  One block per row; the row is staged in shared memory, each warp
// sums whole groups in a fixed order (a single group is summed by all warps, their sums added in
// order), so a row's result depends on nothing but the row.
// All arithmetic is float32; `out` is float32 or bfloat16; weights and the bias are float32.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

// Leaves inv[g] for every group; the caller meets at a barrier before reading them.  With ONE group (the ordinary RMS norm)
// all warps share the sum: every thread adds its columns, then the warps' sums are added in order (`inv[1 ..]` is their room).
__device__ __forceinline__ void group_inverse_rms(const float* vals, float* inv, int width, int groups, float eps) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int part = width / groups;
    if (groups == 1) {
        float sum = 0.0f;
        for (int i = threadIdx.x; i < width; i += kThreads) sum = fmaf(vals[i], vals[i], sum);
        sum = mlr_warp_sum(sum);
        if (lane == 0) inv[1 + warp] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.0f;
            for (int w = 0; w < warps; ++w) total += inv[1 + w];
            inv[0] = 1.0f / sqrtf(total / static_cast<float>(width) + eps);
        }
        return;
    }
    for (int g = warp; g < groups; g += warps) {
        const float* x = vals + static_cast<size_t>(g) * part;
        float sum = 0.0f;
        for (int i = lane; i < part; i += 32) sum = fmaf(x[i], x[i], sum);
        sum = mlr_warp_sum(sum);
        if (lane == 0) inv[g] = 1.0f / sqrtf(sum / static_cast<float>(part) + eps);
    }
}

__device__ __forceinline__ void store4(float* o, int i, float4 v) { *reinterpret_cast<float4*>(o + i) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* o, int i, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(o + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// A contribution that has not been added up yet: row t is  sum_j weights[t, j] * y[row_of_pair[t, j]]  (j = 0 .. top-1 in order)
// + gate[t] * shared[t]  (the results of a token's routed experts, in rows ordered by expert, and of a shared expert).  y null:
// the contribution is `delta` as it stands.
struct Pieces {
    const float* y;
    long long ldy;
    const int* row_of_pair;
    const float* weights;
    int top;
    const float* shared;
    long long ld_shared;
    const float* gate;
};
constexpr int kMaxPieces = 32;

// VEC: four values an access (the width and every row stride are multiples of 4 and the rows start on 16-byte borders); the
// arithmetic and the order of every sum are the same as one value at a time.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) group_rmsnorm_kernel(float* h, const float* delta, int ld_delta, const float* bias,
                                                                 const float* w_post, const float* w_pre, T* out, int ld_out,
                                                                 const int* rows, int width, int groups, float eps, int mode, Pieces pieces) {
    const int norm_delta = mode & 1, plain_out = mode & 2;
    __shared__ float piece_weight[kMaxPieces];
    __shared__ long long piece_from[kMaxPieces];
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    float* vals = reinterpret_cast<float*>(smem);
    float* inv = vals + width;
    const int row = rows ? rows[blockIdx.x] : blockIdx.x;
    const int part = width / groups;
    float* hrow = h + static_cast<size_t>(row) * width;
    constexpr int kStep = VEC ? 4 : 1;
    auto load = [](const float* p, int i) {
        if constexpr (VEC) return __ldcg(reinterpret_cast<const float4*>(p + i));
        else return make_float4(p[i], 0.0f, 0.0f, 0.0f);
    };
    auto keep = [&](int i, float4 v) {
        if constexpr (VEC) *reinterpret_cast<float4*>(vals + i) = v;
        else vals[i] = v.x;
    };
    auto kept = [&](int i) {
        if constexpr (VEC) return *reinterpret_cast<const float4*>(vals + i);
        else return make_float4(vals[i], 0.0f, 0.0f, 0.0f);
    };
    if (delta || pieces.y) {
        const float* d = delta + static_cast<size_t>(row) * ld_delta;
        if (pieces.y) {
            if (threadIdx.x < pieces.top) {
                piece_weight[threadIdx.x] = __ldcg(pieces.weights + static_cast<size_t>(row) * pieces.top + threadIdx.x);
                piece_from[threadIdx.x] = static_cast<long long>(__ldcg(pieces.row_of_pair + static_cast<size_t>(row) * pieces.top + threadIdx.x)) * pieces.ldy;
            }
            __syncthreads();
        }
        const float shared_gate = pieces.y && pieces.shared && pieces.gate ? __ldcg(pieces.gate + row) : 1.0f;
        for (int i = threadIdx.x * kStep; i < width; i += kThreads * kStep) {
            float4 v;
            if (pieces.y) {
                v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int j = 0; j < pieces.top; ++j) {
                    const float4 e = load(pieces.y + piece_from[j], i);
                    const float w = piece_weight[j];
                    v.x = fmaf(w, e.x, v.x); v.y = fmaf(w, e.y, v.y); v.z = fmaf(w, e.z, v.z); v.w = fmaf(w, e.w, v.w);
                }
                if (pieces.shared) {
                    const float4 e = load(pieces.shared + static_cast<size_t>(row) * pieces.ld_shared, i);
                    if (pieces.gate) { v.x = fmaf(shared_gate, e.x, v.x); v.y = fmaf(shared_gate, e.y, v.y); v.z = fmaf(shared_gate, e.z, v.z); v.w = fmaf(shared_gate, e.w, v.w); }
                    else { v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w; }
                }
            } else {
                v = load(d, i);
            }
            if (bias) {
                const float4 b = load(bias, i);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            keep(i, v);
        }
        __syncthreads();
        if (norm_delta) group_inverse_rms(vals, inv, width, groups, eps);
        __syncthreads();
        for (int i = threadIdx.x * kStep; i < width; i += kThreads * kStep) {
            float4 v = kept(i);
            if (norm_delta) {
                v.x *= inv[i / part];
                if constexpr (VEC) { v.y *= inv[(i + 1) / part]; v.z *= inv[(i + 2) / part]; v.w *= inv[(i + 3) / part]; }
            }
            if (w_post) {
                const float4 w = load(w_post, i);
                v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
            }
            const float4 old = load(hrow, i);
            v.x = old.x + v.x; v.y = old.y + v.y; v.z = old.z + v.z; v.w = old.w + v.w;
            if constexpr (VEC) *reinterpret_cast<float4*>(hrow + i) = v;
            else hrow[i] = v.x;
            keep(i, v);
        }
    } else {
        for (int i = threadIdx.x * kStep; i < width; i += kThreads * kStep) keep(i, load(hrow, i));
    }
    if (!out) return;
    T* o = out + static_cast<size_t>(blockIdx.x) * ld_out;
    if (plain_out) {           // every thread wrote the values it reads back
        for (int i = threadIdx.x * kStep; i < width; i += kThreads * kStep) {
            if constexpr (VEC) store4(o, i, kept(i));
            else mlr_store(o, i, vals[i]);
        }
        mlr_grid_dependents_may_start();
        return;
    }
    __syncthreads();
    group_inverse_rms(vals, inv, width, groups, eps);
    __syncthreads();
    for (int i = threadIdx.x * kStep; i < width; i += kThreads * kStep) {
        float4 v = kept(i);
        v.x *= inv[i / part];
        if constexpr (VEC) { v.y *= inv[(i + 1) / part]; v.z *= inv[(i + 2) / part]; v.w *= inv[(i + 3) / part]; }
        if (w_pre) {
            const float4 w = load(w_pre, i);
            v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
        }
        if constexpr (VEC) store4(o, i, v);
        else mlr_store(o, i, v.x);
    }
    mlr_grid_dependents_may_start();
}

}  // namespace

namespace {
int group_rmsnorm(float* h, const float* delta, int ld_delta, const float* bias, const float* w_post, const float* w_pre, void* out, int ld_out,
                  int out_bf16, const int* rows, int count, int width, int groups, float eps, int norm_delta, const Pieces& pieces,
                  cudaStream_t stream) {
    MLR_REQUIRE(count >= 0 && width > 0 && groups > 0 && width % groups == 0,
                "group_rmsnorm: width %d cannot be cut into %d equal groups", width, groups);
    MLR_REQUIRE(eps >= 0.0f, "group_rmsnorm: eps must not be negative");
    MLR_REQUIRE(h && (delta || out || pieces.y), "group_rmsnorm: nothing to do");
    MLR_REQUIRE(!delta || (ld_delta >= width && !rows), "group_rmsnorm: a contribution is added for all rows, with a row stride >= width");
    MLR_REQUIRE(!pieces.y || (!delta && !rows && pieces.top >= 1 && pieces.top <= kMaxPieces && pieces.row_of_pair && pieces.weights &&
                              pieces.ldy >= width && (!pieces.shared || pieces.ld_shared >= width)),
                "group_rmsnorm: a contribution in pieces stands instead of a plain one, for all rows, with at most %d pieces a row", kMaxPieces);
    MLR_REQUIRE(!out || ld_out >= width, "group_rmsnorm: the output's row stride is smaller than the width");
    if (count == 0) return 0;
    const size_t shared = sizeof(float) * (static_cast<size_t>(width) + groups + kThreads / 32);
    MLR_REQUIRE(shared <= 200 * 1024, "group_rmsnorm: a row of %d values does not fit shared memory", width);
    const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = width % 4 == 0 && ld_delta % 4 == 0 && ld_out % 4 == 0 && aligned(h) && aligned(delta) && aligned(bias) && aligned(w_post) &&
                     aligned(w_pre) && aligned(out) && aligned(pieces.y) && pieces.ldy % 4 == 0 && aligned(pieces.shared) && pieces.ld_shared % 4 == 0;
#define MLR_NORM(T, VEC)                                                                                                               \
    do {                                                                                                                               \
        if (shared > 48 * 1024)                                                                                                        \
            cudaFuncSetAttribute(group_rmsnorm_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)); \
        mlr_launch((group_rmsnorm_kernel<T, VEC>), dim3(count), dim3(kThreads), shared, stream, h, delta, ld_delta, bias, w_post, w_pre, \
                   static_cast<T*>(out), ld_out, rows, width, groups, eps, norm_delta, pieces);                                       \
    } while (0)
    if (out_bf16) {
        if (vec) MLR_NORM(__nv_bfloat16, true);
        else MLR_NORM(__nv_bfloat16, false);
    } else {
        if (vec) MLR_NORM(float, true);
        else MLR_NORM(float, false);
    }
#undef MLR_NORM
    return mlr_launched("group_rmsnorm");
}
}  // namespace

MLR_API int mlr_group_rmsnorm(float* h, const float* delta, int ld_delta, const float* bias, const float* w_post,
                              const float* w_pre, void* out, int ld_out, int out_bf16, const int* rows, int count, int width,
                              int groups, float eps, int norm_delta, cudaStream_t stream) {
    return group_rmsnorm(h, delta, ld_delta, bias, w_post, w_pre, out, ld_out, out_bf16, rows, count, width, groups, eps, norm_delta, Pieces{},
                         stream);
}

// The same with the contribution given in pieces (see `Pieces`): what routed experts leave, added up here instead of by a launch
// of its own.  y: float32 rows ordered by expert; row_of_pair, weights: [count, top]; shared: float32 [count, width] or null; gate:
// float32 [count] or null (the shared expert's result then joins as it is).
MLR_API int mlr_group_rmsnorm_pieces(float* h, const float* y, long long ldy, const int* row_of_pair, const float* weights, int top,
                                     const float* shared_y, long long ld_shared, const float* gate, const float* w_post, const float* w_pre,
                                     void* out, int ld_out, int out_bf16, int count, int width, int groups, float eps, int mode,
                                     cudaStream_t stream) {
    MLR_REQUIRE(y, "group_rmsnorm_pieces: no pieces");
    const Pieces pieces = {y, ldy, row_of_pair, weights, top, shared_y, ld_shared, gate};
    return group_rmsnorm(h, nullptr, 0, nullptr, w_post, w_pre, out, ld_out, out_bf16, nullptr, count, width, groups, eps, mode, pieces, stream);
}
