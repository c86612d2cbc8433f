// Layer norm with weight and bias, fused with what a block does to the residual stream around it:
//
//   x   = h[row] + (d1[row] + d2[row] + bias)                 the sub-layers' results, if the block hands any over
//   history[n_prev][row] = x;  x = sum_{j <= n_prev} w[j] * history[j][row]       the depth-weighted average, if asked for
//   h[row] = x                                                                      unless only wanted rows are normed
//   out[r] = (x - mean) / sqrt(var + eps) * weight + bias_n   var = mean of the squared deviations; if a norm is named
//
// `history` holds the stream's earlier states of this step, [states][rows][width] float32, `slot_stride` values apart: state 0
// is what the embedding made, state j + 1 what layer j computed before its own averaging.  A launch with n_prev = 0 and w = {1}
// starts the history (it stores the stream as state 0).  Everything is float32; `out` is float32 or bfloat16.  One block per
// row, the row in shared memory, sums by a fixed tree (a row's result depends on that row only).
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <typename TO>
__global__ void __launch_bounds__(kThreads) depth_norm_kernel(float* h, const float* d1, long long ld1, const float* d2, long long ld2,
                                                              const float* bias, float* history, long long slot_stride, int n_prev,
                                                              const float* dwa, const float* norm_w, const float* norm_b, float eps,
                                                              TO* out, long long ld_out, const int* want_rows, int width, int store_h) {
    mlr_grid_wait();
    extern __shared__ __align__(16) float xs[];       // [width]
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int row = want_rows ? want_rows[r] : r;
    float* hrow = h + static_cast<size_t>(row) * width;
    const bool vec = width % 4 == 0 && ld1 % 4 == 0 && ld2 % 4 == 0 && slot_stride % 4 == 0;
    float sum = 0.0f;
    auto value_at = [&](int c, float x) {
        // x: the stream's value; returns what the stream becomes
        float add = 0.0f;
        bool any = false;
        if (d1) { add = __ldcg(d1 + static_cast<size_t>(row) * ld1 + c); any = true; }
        if (d2) { add += __ldcg(d2 + static_cast<size_t>(row) * ld2 + c); any = true; }
        if (bias) { add += bias[c]; any = true; }
        if (any) x += add;
        if (history) {
            history[static_cast<size_t>(n_prev) * slot_stride + static_cast<size_t>(row) * width + c] = x;
            float mixed = 0.0f;
            for (int j = 0; j < n_prev; ++j)
                mixed = fmaf(dwa[j], __ldcg(history + static_cast<size_t>(j) * slot_stride + static_cast<size_t>(row) * width + c), mixed);
            x = fmaf(dwa[n_prev], x, mixed);
        }
        return x;
    };
    if (vec) {
        for (int c = threadIdx.x * 4; c < width; c += kThreads * 4) {
            float4 x = __ldcg(reinterpret_cast<const float4*>(hrow + c));
            float v[4] = {x.x, x.y, x.z, x.w};
            float add[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            bool any = false;
            if (d1) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(d1 + static_cast<size_t>(row) * ld1 + c));
                add[0] = a.x; add[1] = a.y; add[2] = a.z; add[3] = a.w;
                any = true;
            }
            if (d2) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(d2 + static_cast<size_t>(row) * ld2 + c));
                add[0] += a.x; add[1] += a.y; add[2] += a.z; add[3] += a.w;
                any = true;
            }
            if (bias) {
                const float4 a = *reinterpret_cast<const float4*>(bias + c);
                add[0] += a.x; add[1] += a.y; add[2] += a.z; add[3] += a.w;
                any = true;
            }
            if (any) {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] += add[e];
            }
            if (history) {
                float* slot = history + static_cast<size_t>(row) * width + c;
                *reinterpret_cast<float4*>(slot + static_cast<size_t>(n_prev) * slot_stride) = make_float4(v[0], v[1], v[2], v[3]);
                float mixed[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                int j = 0;
                for (; j + 4 <= n_prev; j += 4) {      // four states on their way at a time
                    float4 s[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) s[u] = __ldcg(reinterpret_cast<const float4*>(slot + static_cast<size_t>(j + u) * slot_stride));
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float w = dwa[j + u];
                        mixed[0] = fmaf(w, s[u].x, mixed[0]); mixed[1] = fmaf(w, s[u].y, mixed[1]);
                        mixed[2] = fmaf(w, s[u].z, mixed[2]); mixed[3] = fmaf(w, s[u].w, mixed[3]);
                    }
                }
                for (; j < n_prev; ++j) {
                    const float4 s = __ldcg(reinterpret_cast<const float4*>(slot + static_cast<size_t>(j) * slot_stride));
                    const float w = dwa[j];
                    mixed[0] = fmaf(w, s.x, mixed[0]); mixed[1] = fmaf(w, s.y, mixed[1]);
                    mixed[2] = fmaf(w, s.z, mixed[2]); mixed[3] = fmaf(w, s.w, mixed[3]);
                }
                const float w = dwa[n_prev];
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = fmaf(w, v[e], mixed[e]);
            }
            if (store_h) *reinterpret_cast<float4*>(hrow + c) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(xs + c) = make_float4(v[0], v[1], v[2], v[3]);
            sum += (v[0] + v[1]) + (v[2] + v[3]);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += kThreads) {
            const float v = value_at(c, __ldcg(hrow + c));
            if (store_h) hrow[c] = v;
            xs[c] = v;
            sum += v;
        }
    }
    mlr_grid_dependents_may_start();
    if (!out) return;
    const float mean = mlr_block_sum(sum, scratch) / static_cast<float>(width);
    float squares = 0.0f;
    for (int c = threadIdx.x; c < width; c += kThreads) {       // the row is whole after the sum's barriers
        const float d = xs[c] - mean;
        squares = fmaf(d, d, squares);
    }
    const float inv = 1.0f / sqrtf(mlr_block_sum(squares, scratch) / static_cast<float>(width) + eps);
    TO* orow = out + static_cast<size_t>(r) * ld_out;
    for (int c = threadIdx.x; c < width; c += kThreads) {
        float v = (xs[c] - mean) * inv * norm_w[c];
        if (norm_b) v += norm_b[c];
        mlr_store(orow, c, v);
    }
}

}  // namespace

// h: float32 [*, width] (row stride width).  d1, d2: float32 results to add (row strides ld1, ld2) or null; bias: float32 [width] or null.
// history: float32 or null; with it, state n_prev is written and the stream becomes the average over states 0..n_prev with the
// weights dwa (float32 [n_prev + 1]).  norm_w, norm_b: float32 [width] (norm_b may be null); out: [rows, width] with row stride
// ld_out in float32 or bfloat16, or null for no norm.  want_rows: int32 [rows] or null (all rows 0..rows-1).
MLR_API int mlr_depth_norm(float* h, const float* d1, long long ld1, const float* d2, long long ld2, const float* bias, float* history,
                           long long slot_stride, int n_prev, const float* dwa, const float* norm_w, const float* norm_b, float eps, void* out,
                           long long ld_out, int out_bf16, const int* want_rows, int rows, int width, int store_h, cudaStream_t stream) {
    MLR_REQUIRE(h && width > 0 && n_prev >= 0, "depth_norm: bad arguments");
    MLR_REQUIRE(!history || (dwa && slot_stride >= 0), "depth_norm: a history needs its weights");
    MLR_REQUIRE(!out || norm_w, "depth_norm: a norm needs its weight");
    MLR_REQUIRE(!(want_rows && (store_h || history)), "depth_norm: a launch over wanted rows leaves the stream as it is");
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(h) % 16 == 0 && reinterpret_cast<uintptr_t>(d1) % 16 == 0 && reinterpret_cast<uintptr_t>(d2) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(history) % 16 == 0 && reinterpret_cast<uintptr_t>(bias) % 16 == 0,
                "depth_norm: buffers must start on 16-byte borders");
    const size_t shared = sizeof(float) * static_cast<size_t>(width);
    MLR_REQUIRE(shared <= 200 * 1024, "depth_norm: a row of %d values does not fit shared memory", width);
    if (rows <= 0) return 0;
    if (out_bf16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(depth_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((depth_norm_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), shared, stream, h, d1, ld1, d2, ld2, bias, history, slot_stride,
                   n_prev, dwa, norm_w, norm_b, eps, static_cast<__nv_bfloat16*>(out), ld_out, want_rows, width, store_h);
    } else {
        if (shared > 48 * 1024) cudaFuncSetAttribute(depth_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((depth_norm_kernel<float>), dim3(rows), dim3(kThreads), shared, stream, h, d1, ld1, d2, ld2, bias, history, slot_stride, n_prev,
                   dwa, norm_w, norm_b, eps, static_cast<float*>(out), ld_out, want_rows, width, store_h);
    }
    return mlr_launched("depth_norm");
}
