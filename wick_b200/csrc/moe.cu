// A mixture of gated experts whose choice is read from a table: token id -> `top` experts,
// each with the same weight.  Expert i: down_i( silu(gate_i x) * (up_i x) ).
//
//   moe_up   : hidden[t][c] = silu(gate x_t) * (up x_t) with the weights of expert table[token_t][c]
//   moe_down : out[t] = base[t] + weight * (down_{e(t,0)} hidden[t][0] + down_{e(t,1)} hidden[t][1] + ...)
//              (choices in table order; base: float32 partial sums of a part that runs for every token)
//
// This form walks the tokens: every (token, choice) reads its expert's matrices (from the L2
// cache when several tokens share an expert).  It is the form of decode steps and of the 32-bit
// path.  Products accumulate in float32 along the inner dimension in a fixed order (lane l takes
// elements l, l + 32, ... or the 8 neighbours at 8 l, 8 l + 256, ...; the 32 sums by the butterfly).
#include "common.cuh"

namespace wick {

template <typename T> __device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int k, int lane) {
    float s = 0.f;
    constexpr int VN = Vec16<T>::N;
    if (k % VN == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int j = lane * VN; j < k; j += 32 * VN) {
            Vec16<T> v;
            v.load(w + j);
#pragma unroll
            for (int i = 0; i < VN; ++i) s = fmaf(v.v[i], x[j + i], s);
        }
    } else {
        for (int j = lane; j < k; j += 32) s = fmaf(ld(w + j), x[j], s);
    }
    return warp_sum(s);
}

constexpr int ROWS_PER_WARP = 4;

// grid (n * top, ceil(ff / (warps * ROWS_PER_WARP))).  gate_up: [experts][2][ff][width] (gate rows, then up rows).
template <typename T>
__global__ void __launch_bounds__(128)
moe_up_kernel(const T* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ table, int top, int n_experts,
              const T* __restrict__ gate_up, T* __restrict__ hidden, int width, int ff) {
    extern __shared__ float xs[];
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    const int t = blockIdx.x / top, c = blockIdx.x - t * top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < width; j += blockDim.x) xs[j] = ld(x + (int64_t)t * width + j);
    __syncthreads();
    const int ex = table[(int64_t)tokens[t] * top + c];
    if (ex < 0 || ex >= n_experts) return;                                   // (a table that names no expert adds nothing)
    const T* wg = gate_up + (int64_t)ex * 2 * ff * width;
    const T* wu = wg + (int64_t)ff * width;
    const int f0 = (blockIdx.y * (blockDim.x >> 5) + warp) * ROWS_PER_WARP;
    for (int f = f0; f < min(f0 + ROWS_PER_WARP, ff); ++f) {
        const float g = dot_row(wg + (int64_t)f * width, xs, width, lane);
        const float u = dot_row(wu + (int64_t)f * width, xs, width, lane);
        if (lane == 0) st(hidden + ((int64_t)t * top + c) * ff + f, g / (1.0f + expf(-g)) * u);
    }
}

// grid (n, ceil(width / (warps * ROWS_PER_WARP))).  down: [experts][width][ff].
template <typename T>
__global__ void __launch_bounds__(128)
moe_down_kernel(const T* __restrict__ hidden, const int* __restrict__ tokens, const int* __restrict__ table, int top,
                int n_experts, const T* __restrict__ down, float weight, const float* __restrict__ base, int base_splits,
                int64_t base_stride, float* __restrict__ out, int width, int ff) {
    extern __shared__ float hs[];                                            // [top][ff]
    pdl_trigger();
    pdl_wait();
    hidden = fresh(hidden);
    base = fresh(base);
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < top * ff; j += blockDim.x) hs[j] = ld(hidden + (int64_t)t * top * ff + j);
    __syncthreads();
    const int o0 = (blockIdx.y * (blockDim.x >> 5) + warp) * ROWS_PER_WARP;
    for (int o = o0; o < min(o0 + ROWS_PER_WARP, width); ++o) {
        float sum = 0.f;
        for (int c = 0; c < top; ++c) {
            const int ex = table[(int64_t)tokens[t] * top + c];
            if (ex < 0 || ex >= n_experts) continue;
            sum += dot_row(down + ((int64_t)ex * width + o) * ff, hs + c * ff, ff, lane);
        }
        if (lane == 0) {
            float v = 0.f;
            for (int s = 0; s < base_splits; ++s) v += base[s * base_stride + (int64_t)t * width + o];
            out[(int64_t)t * width + o] = v + weight * sum;
        }
    }
}

// ---- the form for many tokens: rows sorted by expert ---------------------------------------
// The (token, choice) pairs of a step, numbered t * top + c, are sorted by expert (pairs of one
// expert keep their order), so that every expert's rows lie together and go through an ordinary
// matrix product.  route: expert_of[pair] and counts[expert]; place: row_of[pair] (a warp per
// expert walks all pairs in order and numbers its own); gather: the sorted rows of x; combine:
// out[t] = base[t] + weight * (y[row_of[t, 0]] + y[row_of[t, 1]] + ...), choices in table order.
__global__ void moe_route_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int top, int n_experts,
                                 int* __restrict__ expert_of, int* __restrict__ counts, int n_pairs) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int t = i / top, c = i - t * top;
    int ex = table[(int64_t)tokens[t] * top + c];
    if (ex < 0 || ex >= n_experts) ex = -1;
    expert_of[i] = ex;
    if (ex >= 0) atomicAdd(counts + ex, 1);               // (a count: the order of the additions does not matter)
}

__global__ void __launch_bounds__(32)
moe_place_kernel(const int* __restrict__ expert_of, const int* __restrict__ counts, int* __restrict__ row_of, int n_pairs) {
    pdl_trigger();
    pdl_wait();
    expert_of = fresh(expert_of);
    counts = fresh(counts);
    const int ex = blockIdx.x, lane = threadIdx.x;
    int base = 0;
    for (int e = 0; e < ex; ++e) base += counts[e];
    for (int i0 = 0; i0 < n_pairs; i0 += 32) {
        const int i = i0 + lane;
        const bool mine = i < n_pairs && expert_of[i] == ex;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) row_of[i] = base + __popc(m & ((1u << lane) - 1));
        base += __popc(m);
    }
    if (ex == 0)                                           // pairs without an expert have no row
        for (int i = lane; i < n_pairs; i += 32)
            if (expert_of[i] < 0) row_of[i] = -1;
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ row_of, int top, T* __restrict__ xs, int width) {
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    row_of = fresh(row_of);
    const int pair = blockIdx.x, row = row_of[pair];
    if (row < 0) return;
    const T* src = x + (int64_t)(pair / top) * width;
    T* dst = xs + (int64_t)row * width;
    constexpr int VN = Vec16<T>::N;
    if (width % VN == 0 && (((uintptr_t)x | (uintptr_t)xs) & 15) == 0) {
        for (int j = threadIdx.x * VN; j < width; j += blockDim.x * VN)
            *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(src + j);
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = src[j];
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of, int top, float weight,
                                   const float* __restrict__ base, int base_splits, int64_t base_stride,
                                   float* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    row_of = fresh(row_of);
    base = fresh(base);
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float sum = 0.f;
        for (int c = 0; c < top; ++c) {
            const int row = row_of[t * top + c];
            if (row >= 0) sum += y[(int64_t)row * width + j];
        }
        float v = 0.f;
        for (int s = 0; s < base_splits; ++s) v += base[s * base_stride + (int64_t)t * width + j];
        out[(int64_t)t * width + j] = v + weight * sum;
    }
}

template <typename T>
int moe_up(const void* x, const int* tokens, const int* table, int top, int n_experts, const void* gate_up, void* hidden, int n,
           int width, int ff, cudaStream_t s) {
    WICK_REQUIRE(top > 0 && n_experts > 0 && width > 0 && ff > 0, "moe_up: bad sizes");
    if (n == 0) return 0;
    const int warps = 4;
    WICK_REQUIRE((size_t)width * 4 <= 48 * 1024, "moe_up: width %d is beyond %d", width, 48 * 1024 / 4);
    WICK_CUDA(launch(moe_up_kernel<T>, dim3(n * top, ceil_div(ff, warps * ROWS_PER_WARP)), dim3(warps * 32), (size_t)width * 4, s,
                     (const T*)x, tokens, table, top, n_experts, (const T*)gate_up, (T*)hidden, width, ff));
    return check_launch("moe_up");
}

template <typename T>
int moe_down(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down, float weight,
             const float* base, int base_splits, float* out, int n, int width, int ff, cudaStream_t s) {
    WICK_REQUIRE(top > 0 && n_experts > 0 && width > 0 && ff > 0, "moe_down: bad sizes");
    if (n == 0) return 0;
    const int warps = 4;
    const size_t smem = (size_t)top * ff * 4;
    WICK_REQUIRE(smem <= 48 * 1024, "moe_down: %d choices of %d numbers are beyond one block's shared memory", top, ff);
    WICK_CUDA(launch(moe_down_kernel<T>, dim3(n, ceil_div(width, warps * ROWS_PER_WARP)), dim3(warps * 32), smem, s,
                     (const T*)hidden, tokens, table, top, n_experts, (const T*)down, weight, base, base_splits,
                     (int64_t)n * width, out, width, ff));
    return check_launch("moe_down");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

WICK_API int wick_moe_up_bf16(const void* x, const int* tokens, const int* table, int top, int n_experts, const void* gate_up,
                              void* hidden, int n, int width, int ff, void* s) {
    return moe_up<bf16>(x, tokens, table, top, n_experts, gate_up, hidden, n, width, ff, (cudaStream_t)s);
}
WICK_API int wick_moe_up_f32(const void* x, const int* tokens, const int* table, int top, int n_experts, const void* gate_up,
                             void* hidden, int n, int width, int ff, void* s) {
    return moe_up<float>(x, tokens, table, top, n_experts, gate_up, hidden, n, width, ff, (cudaStream_t)s);
}
WICK_API int wick_moe_down_bf16(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down,
                                float weight, const float* base, int base_splits, float* out, int n, int width, int ff, void* s) {
    return moe_down<bf16>(hidden, tokens, table, top, n_experts, down, weight, base, base_splits, out, n, width, ff, (cudaStream_t)s);
}
WICK_API int wick_moe_down_f32(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down,
                               float weight, const float* base, int base_splits, float* out, int n, int width, int ff, void* s) {
    return moe_down<float>(hidden, tokens, table, top, n_experts, down, weight, base, base_splits, out, n, width, ff,
                           (cudaStream_t)s);
}

// expert_of, row_of: int32 [n * top]; counts: int32 [experts], zero on entry.
WICK_API int wick_moe_route(const int* tokens, const int* table, int top, int n_experts, int* expert_of, int* counts,
                            int* row_of, int n, void* s) {
    WICK_REQUIRE(top > 0 && n_experts > 0 && n >= 0, "moe_route: bad sizes");
    if (n == 0) return 0;
    const int pairs = n * top;
    WICK_CUDA(launch(moe_route_kernel, dim3(ceil_div(pairs, 256)), dim3(256), 0, (cudaStream_t)s, tokens, table, top, n_experts,
                     expert_of, counts, pairs));
    WICK_CUDA(launch(moe_place_kernel, dim3(n_experts), dim3(32), 0, (cudaStream_t)s, (const int*)expert_of, (const int*)counts,
                     row_of, pairs));
    return check_launch("moe_route");
}
WICK_API int wick_moe_gather_bf16(const void* x, const int* row_of, int top, void* xs, int n, int width, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_gather_kernel<bf16>, dim3(n * top), dim3(128), 0, (cudaStream_t)s, (const bf16*)x, row_of, top, (bf16*)xs, width));
    return check_launch("moe_gather");
}
WICK_API int wick_moe_gather_f32(const void* x, const int* row_of, int top, void* xs, int n, int width, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_gather_kernel<float>, dim3(n * top), dim3(128), 0, (cudaStream_t)s, (const float*)x, row_of, top, (float*)xs, width));
    return check_launch("moe_gather");
}
WICK_API int wick_moe_combine(const float* y, const int* row_of, int top, float weight, const float* base, int base_splits,
                              float* out, int n, int width, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_combine_kernel, dim3(n), dim3(256), 0, (cudaStream_t)s, y, row_of, top, weight, base, base_splits,
                     (int64_t)n * width, out, width));
    return check_launch("moe_combine");
}
