// Attention of a prompt's tokens on the tensor cores (bfloat16) for query / key vectors of WICK_DK
// numbers and values of WICK_DV, with keys and values described by strides: a key row may be put
// together from two sources (a part of its own per head and a part all heads share), and a source is
// either the paged cache or a flat array with one row per token of the step (for sequences that
// start at position 0: the keys are then the step's own tokens).
//
// Work partition as in attn_prompt_mma.cu: 64 query rows x one head per block, four warps of 16 rows,
// one tile of 64 keys (a page) per inner step, cp.async two tiles deep, S = Q K^T and O += P V as
// mma.sync m16n8k16 with float32 accumulators, float32 softmax in registers.
//
// Visible to the query at position p: the keys j <= p with p - j < window or j < keep_first (window 0:
// every j <= p).  The tiles a block visits are those that hold kept first keys, then those of the
// window of its rows.  A sink per head joins the denominator.  The result goes out in float32 (for a
// kernel that combines several maps) or in bfloat16 times a gate per (token, head).
#include "common.cuh"

#if !defined(WICK_DK) || !defined(WICK_DV)
#error "compile with -DWICK_DK=<query/key size> -DWICK_DV=<value size>"
#endif

namespace wick {
namespace flex {

constexpr int DK = WICK_DK, DV = WICK_DV;
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK >= 16 && DK <= 256 && DV >= 16 && DV <= 128, "sizes the kernel takes");
constexpr int QT = 64;
constexpr int KCH = DK / 8, VCH = DV / 8;            // 16-byte chunks per row
constexpr bool KSWZ = KCH % 8 == 0, VSWZ = VCH % 8 == 0;
constexpr int KS = DK / 16;                          // k-steps of Q K^T
constexpr int ND = DV / 8;                           // 8-wide blocks of the output row
// Blocks an SM should hold: three where a thread's accumulators are few enough for 170 registers (8 warps an SM leave the
// tensor pipe waiting on every instruction's latency; measured 28 % active), two for the large sizes.
constexpr int MIN_BLOCKS = DK + DV <= 192 ? 3 : 2;
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ int kswz(int row, int chunk) { return KSWZ ? (chunk ^ (row & 7)) : chunk; }
__device__ __forceinline__ int vswz(int row, int chunk) { return VSWZ ? (chunk ^ (row & 7)) : chunk; }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Where the rows of one source lie.  A tile of 64 keys of sequence b, head hv:
//   paged: base + page_table[b][tile] * tile_elems + off(hv) + row * row_stride
//   flat : base + (first token of b + 64 tile + row) * row_stride + off(hv)
// off(hv) = const_off + (hv / hdiv) * hmul + (hv % hmod) * hmul2.   len: numbers of a row that come from here.
struct Source {
    const bf16* base;
    int64_t tile_elems, const_off;
    int hdiv, hmul, hmod, hmul2, row_stride, len, paged;
};

__device__ __forceinline__ const bf16* tile_of(const Source& s, int hv, int b, int tok0, int kt, const int* page_table, int table_width) {
    const int64_t off = s.const_off + (int64_t)(hv / s.hdiv) * s.hmul + (int64_t)(hv % s.hmod) * s.hmul2;
    if (s.paged) return s.base + (int64_t)page_table[(int64_t)b * table_width + kt] * s.tile_elems + off;
    return s.base + ((int64_t)tok0 + (int64_t)kt * kPage) * s.row_stride + off;
}

struct Params {
    const bf16* q;                 // [n, heads, DK]
    Source k0, k1, v;              // a key row: k0.len numbers from k0, then k1.len from k1 (k0.len + k1.len = DK)
    float* out_f32;                // [n, heads, DV], or null
    bf16* out_bf16;                // [n, heads, DV], or null
    const float* gate;             // [n, gate_heads] or null: a factor of the bfloat16 result (head hv -> column hv)
    const float* sink;             // [heads] or null
    const int *cu_seqlens, *start, *page_table;
    int n_seqs, table_width, n_tiles, heads, window, keep_first;
    float scale;
};

__global__ void __launch_bounds__(128, MIN_BLOCKS)
attn_flex_kernel(const Params P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);              // [64][DK]
    bf16* Ks = Qs + QT * DK;                                   // [2][64][DK]
    bf16* Vs = Ks + 2 * kPage * DK;                            // [2][64][DV]
    pdl_trigger();
    pdl_wait();

    const int head = blockIdx.y;
    int b, q0;
    find_work_item(P.cu_seqlens, P.n_seqs, QT, P.n_tiles - 1 - (int)blockIdx.x, b, q0);   // long tiles (late rows of long prompts) first
    if (b < 0) return;
    const int tok0 = P.cu_seqlens[b], q_len = P.cu_seqlens[b + 1] - tok0;
    const int s0 = P.start[b];
    const int rows = min(QT, q_len - q0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kv_len = s0 + q_len;
    const int p_first = s0 + q0, p_last = s0 + q0 + rows - 1;
    const int window = P.window, keep = P.window > 0 ? P.keep_first : 0;
    // the tiles this block visits: those with kept first keys that lie before the window's first tile, then the window's
    const int kt_lo = window > 0 ? max(0, p_first - window + 1) / kPage : 0;
    const int kt_hi = p_last / kPage;
    const int n_kept = min(kt_lo, (keep + kPage - 1) / kPage);
    const int n_visit = n_kept + (kt_hi - kt_lo + 1);
    auto tile_index = [&](int i) { return i < n_kept ? i : kt_lo + (i - n_kept); };

    auto load_tiles = [&](int i) {
        const int kt = tile_index(i), buf = i & 1;
        const int valid = kv_len - kt * kPage;                  // rows of the tile that hold a token
        const bf16* p0 = tile_of(P.k0, head, b, tok0, kt, P.page_table, P.table_width);
        const bf16* p1 = P.k1.len ? tile_of(P.k1, head, b, tok0, kt, P.page_table, P.table_width) : nullptr;
        const bf16* pv = tile_of(P.v, head, b, tok0, kt, P.page_table, P.table_width);
        bf16* kd = Ks + buf * kPage * DK;
        bf16* vd = Vs + buf * kPage * DV;
        const int c0 = P.k0.len >> 3;
        for (int x = tid; x < kPage * KCH; x += 128) {
            const int row = x / KCH, c = x % KCH;
            const int src_row = min(row, max(valid, 1) - 1);    // (an address inside the array also for rows that are zero-filled)
            const bf16* src = c < c0 ? p0 + (int64_t)src_row * P.k0.row_stride + c * 8 : p1 + (int64_t)src_row * P.k1.row_stride + (c - c0) * 8;
            cp_async16(kd + row * DK + kswz(row, c) * 8, src, row < valid);
        }
        for (int x = tid; x < kPage * VCH; x += 128) {
            const int row = x / VCH, c = x % VCH;
            const int src_row = min(row, max(valid, 1) - 1);
            cp_async16(vd + row * DV + vswz(row, c) * 8, pv + (int64_t)src_row * P.v.row_stride + c * 8, row < valid);
        }
    };

    // query tile (rows past the end repeat the last valid row) and the first key/value tile
    for (int x = tid; x < QT * KCH; x += 128) {
        const int row = x / KCH, c = x % KCH;
        const int src_row = min(row, rows - 1);
        cp_async16(Qs + row * DK + kswz(row, c) * 8, P.q + ((int64_t)(tok0 + q0 + src_row) * P.heads + head) * DK + c * 8, true);
    }
    load_tiles(0);
    cp_async_commit();

    // per-thread rows: r_lo = 16 warp + lane / 4, r_hi = r_lo + 8
    const int r_lo = warp * 16 + (lane >> 2);
    const int pos_lo = s0 + q0 + min(r_lo, rows - 1), pos_hi = s0 + q0 + min(r_lo + 8, rows - 1);
    const int vis_lo = window > 0 ? pos_lo - window + 1 : 0, vis_hi = window > 0 ? pos_hi - window + 1 : 0;   // first key of the window
    const float sl2 = P.scale * 1.4426950408889634f;            // scores in units of log2(e)
    const float sink2 = P.sink ? P.sink[head] * 1.4426950408889634f : -INFINITY;

    float o[ND][4];
#pragma unroll
    for (int d = 0; d < ND; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_lo = sink2, m_hi = sink2, l_lo = 0.f, l_hi = 0.f;

    for (int i = 0; i < n_visit; ++i) {
        const int buf = i & 1, kt = tile_index(i);
        if (i + 1 < n_visit) {                                  // prefetch the next tile into the other buffer
            load_tiles(i + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* Kb = Ks + buf * kPage * DK;
        const bf16* Vb = Vs + buf * kPage * DV;

        // ---- S = Q K^T for 64 keys: 8 blocks of 8 keys ----
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t qf[4];
            const int qrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(qf, Qs + qrow * DK + kswz(qrow, 2 * ks + (lane >> 4)) * 8);
#pragma unroll
            for (int nb = 0; nb < 8; nb += 2) {
                uint32_t kf[4];
                const int key = 8 * (nb + (lane >> 4)) + (lane & 7);
                ldmatrix_x4(kf, Kb + key * DK + kswz(key, 2 * ks + ((lane >> 3) & 1)) * 8);
                mma16816(s[nb], qf, kf[0], kf[1]);
                mma16816(s[nb + 1], qf, kf[2], kf[3]);
            }
        }
        // ---- mask, running maximum, probabilities ----
        const int key0 = kt * kPage + (lane & 3) * 2;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + nb * 8 + e;
                float a = s[nb][e] * sl2, c = s[nb][2 + e] * sl2;
                if (key > pos_lo || (key < vis_lo && key >= keep)) a = -INFINITY;
                if (key > pos_hi || (key < vis_hi && key >= keep)) c = -INFINITY;
                s[nb][e] = a;
                s[nb][2 + e] = c;
                mx_lo = fmaxf(mx_lo, a);
                mx_hi = fmaxf(mx_hi, c);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        // (a row may see nothing of a tile: its maximum stays -inf, and exponents are then taken against 0)
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float rf_lo = mn_lo == -INFINITY ? 0.f : mn_lo, rf_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float c_lo = exp2f(m_lo - rf_lo), c_hi = exp2f(m_hi - rf_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nb][e] = exp2f(s[nb][e] - rf_lo);
                s[nb][2 + e] = exp2f(s[nb][2 + e] - rf_hi);
                sum_lo += s[nb][e];
                sum_hi += s[nb][2 + e];
            }
        }
        l_lo = l_lo * c_lo + sum_lo;                            // per-thread partial denominators; joined at the end
        l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
        for (int d = 0; d < ND; ++d) {
            o[d][0] *= c_lo; o[d][1] *= c_lo;
            o[d][2] *= c_hi; o[d][3] *= c_hi;
        }
        // ---- O += P V: 4 steps of 16 keys ----
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
            pf[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
            pf[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
            pf[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {
                uint32_t vf[4];
                const int key = 16 * j + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(vf, Vb + key * DV + vswz(key, nd + (lane >> 4)) * 8);
                mma16816(o[nd], pf, vf[0], vf[1]);
                mma16816(o[nd + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();                                        // everyone is done with this buffer
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (P.sink) {                                               // (every row sees itself: its maximum is finite by now)
        l_lo += exp2f(sink2 - m_lo);
        l_hi += exp2f(sink2 - m_hi);
    }
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = r_lo + 8 * half;
        if (r >= rows) continue;
        const int64_t t = tok0 + q0 + r;
        float inv = 1.0f / (half ? l_hi : l_lo);
        if (P.out_f32) {
            float* op = P.out_f32 + (t * P.heads + head) * DV + col;
#pragma unroll
            for (int d = 0; d < ND; ++d) *reinterpret_cast<float2*>(op + d * 8) = make_float2(o[d][2 * half] * inv, o[d][2 * half + 1] * inv);
        } else {
            if (P.gate) inv *= P.gate[t * P.heads + head];
            bf16* op = P.out_bf16 + (t * P.heads + head) * DV + col;
#pragma unroll
            for (int d = 0; d < ND; ++d) *reinterpret_cast<uint32_t*>(op + d * 8) = pack_bf16(o[d][2 * half] * inv, o[d][2 * half + 1] * inv);
        }
    }
}

// y[t, h] = a_1 - lambda a_2 over the two maps' results a [n, H, 2, e] (float32), then y / sqrt(mean(y^2) + eps) * factor,
// in bfloat16: one warp per (token, head).
__global__ void __launch_bounds__(128)
combine_maps_kernel(const float* __restrict__ a, bf16* __restrict__ out, int64_t n_heads, int e, float lam, float eps, float factor) {
    pdl_trigger();
    pdl_wait();
    a = fresh(a);
    const int lane = threadIdx.x & 31;
    const int64_t th = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (th >= n_heads) return;
    const float* a1 = a + th * 2 * e;
    const float* a2 = a1 + e;
    float y[DV / 32 + 1], ss = 0.f;
#pragma unroll
    for (int c = 0; c < DV / 32 + 1; ++c) {
        const int x = lane + 32 * c;
        y[c] = x < e ? a1[x] - lam * a2[x] : 0.f;
        ss = fmaf(y[c], y[c], ss);
    }
    ss = warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / (float)e + eps);
#pragma unroll
    for (int c = 0; c < DV / 32 + 1; ++c) {
        const int x = lane + 32 * c;
        if (x < e) out[th * e + x] = __float2bfloat16_rn((y[c] * f) * factor);
    }
}

}  // namespace flex
}  // namespace wick

using namespace wick;

WICK_API int wick_attn_flex_sizes(int* dk, int* dv) {
    *dk = flex::DK;
    *dv = flex::DV;
    return 0;
}

// src: three sources (key part 0, key part 1, values) of ten numbers each, as 64-bit integers:
//   address, tile_elems, const_off, hdiv, hmul, hmod, hmul2, row_stride, len, paged.
WICK_API int wick_attn_flex_bf16(const void* q, const int64_t* src, void* out_f32, void* out_bf16, const float* gate, const float* sink,
                                 const int* cu_seqlens, int n_seqs, const int* start, const int* page_table, int table_width,
                                 int n_tiles, int heads, int window, int keep_first, float scale, void* s) {
    using namespace flex;
    Params P;
    P.q = (const bf16*)q;
    Source* dst[3] = {&P.k0, &P.k1, &P.v};
    for (int i = 0; i < 3; ++i) {
        const int64_t* a = src + 10 * i;
        Source& S = *dst[i];
        S.base = (const bf16*)(uintptr_t)a[0];
        S.tile_elems = a[1];
        S.const_off = a[2];
        S.hdiv = (int)a[3]; S.hmul = (int)a[4]; S.hmod = (int)a[5]; S.hmul2 = (int)a[6];
        S.row_stride = (int)a[7]; S.len = (int)a[8]; S.paged = (int)a[9];
        WICK_REQUIRE(S.hdiv > 0 && S.hmod > 0, "attn_flex: a source's head divisors must be positive");
        WICK_REQUIRE(S.len == 0 || (((uintptr_t)S.base) % 16 == 0 && S.row_stride % 8 == 0 && S.const_off % 8 == 0 && S.hmul % 8 == 0 &&
                                    S.hmul2 % 8 == 0 && S.tile_elems % 8 == 0 && S.len % 8 == 0),
                     "attn_flex: a source's rows must start at multiples of 16 bytes");
    }
    WICK_REQUIRE(P.k0.len + P.k1.len == DK && P.k0.len > 0, "attn_flex: key parts of %d + %d numbers, the kernel was built for %d",
                 P.k0.len, P.k1.len, DK);
    WICK_REQUIRE(P.v.len == DV, "attn_flex: values of %d numbers, the kernel was built for %d", P.v.len, DV);
    WICK_REQUIRE((out_f32 == nullptr) != (out_bf16 == nullptr), "attn_flex: one place for the result");
    WICK_REQUIRE(heads > 0 && heads <= 65535 && window >= 0 && keep_first >= 0, "attn_flex: bad head count or window");
    P.out_f32 = (float*)out_f32;
    P.out_bf16 = (bf16*)out_bf16;
    P.gate = gate;
    P.sink = sink;
    P.cu_seqlens = cu_seqlens; P.start = start; P.page_table = page_table;
    P.n_seqs = n_seqs; P.table_width = table_width; P.n_tiles = n_tiles; P.heads = heads; P.window = window; P.keep_first = keep_first;
    P.scale = scale;
    if (n_tiles == 0) return 0;
    const size_t smem = ((size_t)(QT + 2 * kPage) * DK + 2 * kPage * DV) * sizeof(bf16);
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        WICK_CUDA(cudaFuncSetAttribute(attn_flex_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised = true;
    }
    WICK_CUDA(launch(attn_flex_kernel, dim3(n_tiles, heads), dim3(128), smem, (cudaStream_t)s, P));
    return check_launch("attn_flex");
}

WICK_API int wick_combine_maps_bf16(const float* a, void* out, int64_t n_heads, int e, float lam, float eps, float factor, void* s) {
    WICK_REQUIRE(e > 0 && e <= flex::DV, "combine_maps: values of %d numbers, built for %d", e, flex::DV);
    if (n_heads == 0) return 0;
    WICK_CUDA(launch(flex::combine_maps_kernel, dim3(ceil_div(n_heads, 4)), dim3(128), 0, (cudaStream_t)s, a, (flex::bf16*)out, n_heads, e,
                     lam, eps, factor));
    return check_launch("combine_maps");
}
