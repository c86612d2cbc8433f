// Attention whose keys and values are projections of ONE small vector per token (the latent), so that
// only that vector is cached:  k_h = Uk_h c,  v_h = Uv_h c.
//
// The scores  q_h . (Uk_h c)  equal  (Uk_h^T q_h) . c,  and  sum_j p_j Uv_h c_j = Uv_h (sum_j p_j c_j):  with the
// query taken through Uk_h^T first and the result through Uv_h afterwards, attention runs on the cached latents
// themselves, as keys and as values of one shared kv head (`attention_masked.cu` with shared_kv).  Here are the
// two row-wise pieces around it:
//
//   mlr_latent_cache    c = rmsnorm(row of the down projection) * weight, float32 math, into the token's place
//                       of its page ([page][token_in_page][rank], one kv head, keys only)
//   mlr_head_project    y[m, h, :] = x[m, h, :] W_h,  W [heads, A, B] row-major, float32 sums in the order a = 0..A-1 (the
//                       float32 path and odd sizes; bfloat16 rows on 16-byte borders take `mlr_batched_product_bf16` of experts.cu)
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kRows = 8;

template <typename T>
__global__ void __launch_bounds__(kThreads) latent_cache_kernel(const T* in, long long ld, const T* weight_t, const float* weight_f, float eps,
                                                                int rank, T* cache, int num_pages, const int* positions,
                                                                const int* segment_of_row, const int* block_table, int table_stride,
                                                                int page_size, int* status) {
    mlr_grid_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const int position = positions[row];
    const int page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
        return;
    }
    const T* x = in + static_cast<size_t>(row) * ld;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < rank; c += kThreads) {
        const float v = mlr_load(x, c);
        sum = fmaf(v, v, sum);
    }
    const float inv = 1.0f / sqrtf(mlr_block_sum(sum, scratch) / static_cast<float>(rank) + eps);
    T* dst = cache + (static_cast<size_t>(page) * page_size + position % page_size) * rank;
    for (int c = threadIdx.x; c < rank; c += kThreads) {
        const float w = weight_f ? weight_f[c] : mlr_load(weight_t, c);
        mlr_store(dst, c, mlr_load(x, c) * inv * w);
    }
    mlr_grid_dependents_may_start();
}

// The latent with a rotated key part beside it.  A row of the down projection holds `rank` values (normed into the latent) and then
// `rot` values that all heads share as the rotated part of their keys; the cache row of a token is [latent | rotated part].  The queries'
// own rotated parts (head h's at column q_first + h * q_step of `q`) are turned by the same angles and written behind the place of
// that head's projected query in `qout` (column qo_first + h * qo_step).  Of the `rot` values the first `rot_dims` turn by
// position * freq[i], float32, value 2i with value 2i + 1 (`interleaved`) or value i with value i + rot_dims / 2; the rest pass.
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_rot_cache_kernel(const T* in, long long ld, const float* weight, float eps, int rank, int rot,
                                                                    int rot_dims, int interleaved, const float* freq, const T* q, long long ldq,
                                                                    int q_first, int q_step, int heads, T* qout, long long ldqo, int qo_first,
                                                                    int qo_step, T* cache, int num_pages, const int* positions,
                                                                    const int* segment_of_row, const int* block_table, int table_stride,
                                                                    int page_size, int write_cache, int* status) {
    mlr_grid_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const int position = positions[row];
    const float p = static_cast<float>(position);
    const int half = rot_dims / 2;
    // value c of a rotated part whose values are read by `at`
    auto turned = [&](auto at, int c) {
        float value = at(c);
        if (c < rot_dims) {
            const int pair = interleaved ? c >> 1 : (c < half ? c : c - half);
            const bool first = interleaved ? !(c & 1) : c < half;
            const int mate = interleaved ? c ^ 1 : (c < half ? c + half : c - half);
            float sn, cs;
            sincosf(p * freq[pair], &sn, &cs);
            const float other = at(mate);
            value = first ? value * cs - other * sn : value * cs + other * sn;
        }
        return value;
    };
    for (int i = threadIdx.x; i < heads * rot; i += kThreads) {
        const int head = i / rot, c = i % rot;
        const T* src = q + static_cast<size_t>(row) * ldq + q_first + static_cast<size_t>(head) * q_step;
        mlr_store(qout + static_cast<size_t>(row) * ldqo + qo_first + static_cast<size_t>(head) * qo_step, c,
                  turned([&](int k) { return mlr_load(src, k); }, c));
    }
    if (!write_cache) return;
    const int page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
        return;
    }
    const T* x = in + static_cast<size_t>(row) * ld;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < rank; c += kThreads) {
        const float v = mlr_load(x, c);
        sum = fmaf(v, v, sum);
    }
    const float inv = 1.0f / sqrtf(mlr_block_sum(sum, scratch) / static_cast<float>(rank) + eps);
    T* dst = cache + (static_cast<size_t>(page) * page_size + position % page_size) * (rank + rot);
    for (int c = threadIdx.x; c < rank; c += kThreads) mlr_store(dst, c, mlr_load(x, c) * inv * weight[c]);
    for (int c = threadIdx.x; c < rot; c += kThreads) mlr_store(dst, rank + c, turned([&](int k) { return mlr_load(x, rank + k); }, c));
    mlr_grid_dependents_may_start();
}

// A block: kRows rows x one head x 128 outputs; the rows' inputs of that head as float32 in shared memory.
template <typename T>
__global__ void __launch_bounds__(kThreads) head_project_kernel(const T* x, long long ldx, const T* w, T* y, long long ldy, int rows, int A, int B,
                                                                int x_step, int y_step) {
    mlr_grid_wait();
    extern __shared__ __align__(16) float xs[];          // [kRows][A]
    const int row0 = blockIdx.x * kRows, head = blockIdx.y, b = blockIdx.z * kThreads + threadIdx.x;
    const int n = min(kRows, rows - row0);
    for (int i = threadIdx.x; i < kRows * A; i += kThreads) {
        const int r = i / A, a = i % A;
        xs[i] = r < n ? mlr_load(x + static_cast<size_t>(row0 + r) * ldx + static_cast<size_t>(head) * x_step, a) : 0.0f;
    }
    __syncthreads();
    mlr_grid_dependents_may_start();
    if (b >= B) return;
    const T* wh = w + static_cast<size_t>(head) * A * B + b;
    float acc[kRows] = {};
    int a = 0;
    for (; a + 8 <= A; a += 8) {          // eight loads of the matrix in flight
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = mlr_load(wh, static_cast<size_t>(a + i) * B);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int r = 0; r < kRows; ++r) acc[r] = fmaf(xs[r * A + a + i], v[i], acc[r]);
    }
    for (; a < A; ++a) {
        const float v = mlr_load(wh, static_cast<size_t>(a) * B);
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r] = fmaf(xs[r * A + a], v, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r)
        if (r < n) mlr_store(y + static_cast<size_t>(row0 + r) * ldy + static_cast<size_t>(head) * y_step, b, acc[r]);
}

}  // namespace

// in: the rows of the down projection (row stride ld, `rank` values each); weight: [rank] in float32 (weight_f32) or the
// activations' precision; cache: [pages, page_size * rank] of the activations' precision.
MLR_API int mlr_latent_cache(const void* in, long long ld, int act_bf16, const void* weight, int weight_f32, float eps, int rank, void* cache,
                             int num_pages, const int* positions, const int* segment_of_row, const int* block_table, int table_stride,
                             int page_size, int rows, int* status, cudaStream_t stream) {
    MLR_REQUIRE(in && weight && cache && positions && segment_of_row && block_table && rank > 0 && page_size > 0 && num_pages > 0,
                "latent_cache: bad arguments");
    if (rows <= 0) return 0;
    const float* wf = weight_f32 ? static_cast<const float*>(weight) : nullptr;
    if (act_bf16)
        mlr_launch((latent_cache_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const __nv_bfloat16*>(in), ld,
                   static_cast<const __nv_bfloat16*>(weight), wf, eps, rank, static_cast<__nv_bfloat16*>(cache), num_pages, positions,
                   segment_of_row, block_table, table_stride, page_size, status);
    else
        mlr_launch((latent_cache_kernel<float>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const float*>(in), ld,
                   static_cast<const float*>(weight), wf, eps, rank, static_cast<float*>(cache), num_pages, positions, segment_of_row,
                   block_table, table_stride, page_size, status);
    return mlr_launched("latent_cache");
}

// in: rows of the down projection, [rank | rot] values each (row stride ld); weight: float32 [rank]; freq: float32 [rot_dims / 2];
// cache: [pages, page_size * (rank + rot)] of the activations' precision (with write_cache 0 only the queries are turned).
MLR_API int mlr_latent_rot_cache(const void* in, long long ld, int act_bf16, const float* weight, float eps, int rank, int rot, int rot_dims,
                                 int interleaved, const float* freq, const void* q, long long ldq, int q_first, int q_step, int heads, void* qout,
                                 long long ldqo, int qo_first, int qo_step, void* cache, int num_pages, const int* positions,
                                 const int* segment_of_row, const int* block_table, int table_stride, int page_size, int write_cache, int rows,
                                 int* status, cudaStream_t stream) {
    MLR_REQUIRE(positions && q && qout && rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && (rot_dims == 0 || freq) &&
                    heads > 0, "latent_rot_cache: bad arguments");
    MLR_REQUIRE(!write_cache || (in && weight && cache && segment_of_row && block_table && page_size > 0 && num_pages > 0),
                "latent_rot_cache: writing the cache needs the projection, the norm's weight and the cache");
    if (rows <= 0) return 0;
    if (act_bf16)
        mlr_launch((latent_rot_cache_kernel<__nv_bfloat16>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const __nv_bfloat16*>(in), ld, weight,
                   eps, rank, rot, rot_dims, interleaved, freq, static_cast<const __nv_bfloat16*>(q), ldq, q_first, q_step, heads,
                   static_cast<__nv_bfloat16*>(qout), ldqo, qo_first, qo_step, static_cast<__nv_bfloat16*>(cache), num_pages, positions,
                   segment_of_row, block_table, table_stride, page_size, write_cache, status);
    else
        mlr_launch((latent_rot_cache_kernel<float>), dim3(rows), dim3(kThreads), 0, stream, static_cast<const float*>(in), ld, weight, eps, rank, rot,
                   rot_dims, interleaved, freq, static_cast<const float*>(q), ldq, q_first, q_step, heads, static_cast<float*>(qout), ldqo, qo_first,
                   qo_step, static_cast<float*>(cache), num_pages, positions, segment_of_row, block_table, table_stride, page_size, write_cache, status);
    return mlr_launched("latent_rot_cache");
}

// x: [rows, heads * x_step] (row stride ldx; head h's A inputs start at column h * x_step), w: [heads, A, B], y: [rows, heads * y_step]
// (row stride ldy; head h's B outputs start at column h * y_step), all in the activations' precision.
MLR_API int mlr_head_project_strided(const void* x, long long ldx, int x_step, const void* w, void* y, long long ldy, int y_step, int act_bf16, int rows,
                                     int heads, int A, int B, cudaStream_t stream) {
    MLR_REQUIRE(x && w && y && heads > 0 && heads <= 65535 && A > 0 && B > 0 && x_step >= A && y_step >= B, "head_project: bad arguments");
    const size_t shared = sizeof(float) * kRows * static_cast<size_t>(A);
    MLR_REQUIRE(shared <= 200 * 1024, "head_project: %d inputs per head do not fit shared memory", A);
    if (rows <= 0) return 0;
    const dim3 grid((rows + kRows - 1) / kRows, heads, (B + kThreads - 1) / kThreads);
    if (act_bf16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(head_project_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((head_project_kernel<__nv_bfloat16>), dim3(grid), dim3(kThreads), shared, stream, static_cast<const __nv_bfloat16*>(x), ldx,
                   static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), ldy, rows, A, B, x_step, y_step);
    } else {
        if (shared > 48 * 1024) cudaFuncSetAttribute(head_project_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        mlr_launch((head_project_kernel<float>), dim3(grid), dim3(kThreads), shared, stream, static_cast<const float*>(x), ldx,
                   static_cast<const float*>(w), static_cast<float*>(y), ldy, rows, A, B, x_step, y_step);
    }
    return mlr_launched("head_project");
}

// The same with the heads' inputs and outputs side by side (x_step = A, y_step = B).
MLR_API int mlr_head_project(const void* x, long long ldx, const void* w, void* y, long long ldy, int act_bf16, int rows, int heads, int A, int B,
                             cudaStream_t stream) {
    return mlr_head_project_strided(x, ldx, A, w, y, ldy, B, act_bf16, rows, heads, A, B, stream);
}
