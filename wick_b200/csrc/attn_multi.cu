// Attention whose heads hold more than one score map, over paged storage described by
// strides, and the kernels around attention through a cached latent.
//
//   attend   : every new token over the cache.  A query head holds MAPS vectors of dm numbers;
//              map a scores the a-th dm numbers of the key row, has a softmax of its own, and
//              weighs the SAME value rows.  Visible keys of the query at position p: with a
//              window, the keys j <= p with p - j < window or j < keep_first; else every j <= p.
//              A sink per head joins a map's denominator.  MAPS = 2 ends with
//              y = y_1 - lambda y_2, y / sqrt(mean(y^2) + eps) * factor over the head's values.
//              Where a key row and a value row lie in a page is given by strides, so the same
//              kernel reads pages of [kv head][64][d] keys followed by [kv head][64][e] values
//              and pages of [64][row] rows whose first e numbers are the value.
//   finish   : (latent) the down-projection's float32 partial sums -> the normed query latent,
//              the position's cache row (normed latent, turned key part) and the heads' gates
//   absorb   : (latent) q_lat[t, h] = [Wuk_h^T q_flat[t, h] | turned q_rot[t, h]]
//   expand   : (latent) out[t, h] = gate[t, h] * Wuv_h y[t, h]
//
// Scores, softmax, weights, sums and norms are float32.  A token's arithmetic does not depend
// on what else the step holds, up to the number of warps that share its keys.
#include "common.cuh"

namespace wick {

constexpr int MV_CHUNKS = 4;                    // value sizes up to 512: a lane holds 4 neighbours of every 128

__device__ __forceinline__ void mv_load4(const float* p, float* v) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void mv_load4(const __nv_bfloat16* p, float* v) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// The v-th visible key (v counts the kept first keys, then the window).
__device__ __forceinline__ int visible_key(int v, int n_kept, int lo) { return v < n_kept ? v : lo + (v - n_kept); }

// One block per (token, query head); its warps share the visible keys, 32 at a time.  In a tile,
// lane l scores key l of the tile for every map (dot products in index order), the running maximum
// and sum of each map follow, then every lane adds the tile's weighted value rows into its own
// elements of each map's result.  The warps' partial results are folded in warp order by warp 0.
template <typename T, typename TQ, typename TO, int MAPS>
__global__ void __launch_bounds__(256)
attn_multi_kernel(const TQ* __restrict__ q, const T* __restrict__ store, TO* __restrict__ out,
                  const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                  const int* __restrict__ page_table, int table_width, int H, int G, int dm, int e, int64_t page_elems,
                  int k_row, int64_t v_off, int v_row, float scale, int window, int keep_first,
                  const float* __restrict__ sink, float lam, float eps, float factor) {
    extern __shared__ float smem[];
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    store = fresh(store);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int t = blockIdx.x / H, h = blockIdx.x - t * H;
    const int g = h / (H / G);
    const int pos = positions[t];
    const int* table = page_table + (int64_t)seq_of_token[t] * table_width;
    const int d = MAPS * dm, d_pad = (d + 3) & ~3, e_pad = (e + 127) / 128 * 128;
    float* qs = smem;                           // [d]
    float* ms = qs + d_pad;                     // [warps][MAPS] maxima, then [warps][MAPS] sums
    float* accs = ms + 2 * MAPS * n_warps;      // [warps][MAPS][e_pad]
    for (int x = threadIdx.x; x < d; x += blockDim.x) qs[x] = ld(q + ((int64_t)t * H + h) * d + x);
    __syncthreads();
    constexpr int VN = Vec16<T>::N;
    const bool base_ok = (((uintptr_t)store) & 15) == 0;
    const bool k_vec = base_ok && dm % VN == 0 && k_row % VN == 0 && page_elems % VN == 0;
    const bool v_vec = base_ok && e % 4 == 0 && v_row % 4 == 0 && page_elems % 4 == 0 && v_off % 4 == 0;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_kept = window > 0 ? min(keep_first, lo) : 0;
    const int total = n_kept + (pos - lo + 1);
    float m[MAPS], l[MAPS], acc[MAPS][4 * MV_CHUNKS];
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) acc[a][c] = 0.f;
    }
    for (int v0 = 32 * warp; v0 < total; v0 += 32 * n_warps) {
        const int vi = v0 + lane;
        const bool valid = vi < total;
        float s[MAPS], p[MAPS];
#pragma unroll
        for (int a = 0; a < MAPS; ++a) s[a] = -INFINITY;
        if (valid) {
            const int key = visible_key(vi, n_kept, lo);
            const T* kp = store + (int64_t)table[key / kPage] * page_elems + ((int64_t)g * kPage + (key % kPage)) * k_row;
#pragma unroll
            for (int a = 0; a < MAPS; ++a) {
                const float* qa = qs + a * dm;
                const T* ka = kp + a * dm;
                float dot = 0.f;
                if (k_vec) {
                    for (int x = 0; x < dm; x += 2 * VN) {           // two loads of 16 bytes in flight
                        Vec16<T> kk[2];
                        kk[0].load(ka + x);
                        if (x + VN < dm) kk[1].load(ka + x + VN);
#pragma unroll
                        for (int i = 0; i < VN; ++i) dot = fmaf(qa[x + i], kk[0].v[i], dot);
                        if (x + VN < dm) {
#pragma unroll
                            for (int i = 0; i < VN; ++i) dot = fmaf(qa[x + VN + i], kk[1].v[i], dot);
                        }
                    }
                } else {
                    for (int x = 0; x < dm; ++x) dot = fmaf(qa[x], ld(ka + x), dot);
                }
                s[a] = dot * scale;
            }
        }
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            const float m_new = fmaxf(m[a], warp_max(s[a]));         // finite: the tile's first key is visible
            const float corr = expf(m[a] - m_new);                   // (m = -inf at first: 0)
            p[a] = valid ? expf(s[a] - m_new) : 0.f;
            l[a] = l[a] * corr + warp_sum(p[a]);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < 4 * MV_CHUNKS; ++c) acc[a][c] *= corr;
        }
        const int n_keys = min(32, total - v0);
        for (int jj = 0; jj < n_keys; ++jj) {
            const int key = visible_key(v0 + jj, n_kept, lo);
            const T* vp = store + (int64_t)table[key / kPage] * page_elems + v_off + ((int64_t)g * kPage + (key % kPage)) * v_row;
            float pj[MAPS];
#pragma unroll
            for (int a = 0; a < MAPS; ++a) pj[a] = __shfl_sync(0xffffffffu, p[a], jj);
#pragma unroll
            for (int c = 0; c < MV_CHUNKS; ++c) {
                const int x = 128 * c + 4 * lane;
                if (x < e) {
                    float vv[4];
                    if (v_vec) {
                        mv_load4(vp + x, vv);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) vv[i] = x + i < e ? ld(vp + x + i) : 0.f;
                    }
#pragma unroll
                    for (int a = 0; a < MAPS; ++a)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[a][4 * c + i] = fmaf(pj[a], vv[i], acc[a][4 * c + i]);
                }
            }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            ms[warp * MAPS + a] = m[a];
            ms[(n_warps + warp) * MAPS + a] = l[a];
        }
    }
#pragma unroll
    for (int a = 0; a < MAPS; ++a)
#pragma unroll
        for (int c = 0; c < MV_CHUNKS; ++c)
            if (128 * c < e_pad)
#pragma unroll
                for (int i = 0; i < 4; ++i) accs[((int64_t)warp * MAPS + a) * e_pad + 128 * c + 4 * lane + i] = acc[a][4 * c + i];
    __syncthreads();
    if (warp != 0) return;
    // warp 0 folds the warps' results, map by map; a lane holds its elements of the head's result
    float y[MAPS][4 * MV_CHUNKS];
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
        float big = sink ? sink[h] : -INFINITY;
        for (int w = 0; w < n_warps; ++w) big = fmaxf(big, ms[w * MAPS + a]);      // finite: warp 0 holds a visible key
        float sum = sink ? expf(sink[h] - big) : 0.f;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[a][c] = 0.f;
        for (int w = 0; w < n_warps; ++w) {
            const float mw = ms[w * MAPS + a];
            const float f = mw == -INFINITY ? 0.f : expf(mw - big);
            sum += ms[(n_warps + w) * MAPS + a] * f;
#pragma unroll
            for (int c = 0; c < MV_CHUNKS; ++c)
                if (128 * c < e_pad)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        y[a][4 * c + i] = fmaf(accs[((int64_t)w * MAPS + a) * e_pad + 128 * c + 4 * lane + i], f, y[a][4 * c + i]);
        }
        const float inv = 1.0f / sum;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[a][c] *= inv;
    }
    TO* o = out + ((int64_t)t * H + h) * e;
    if (MAPS == 2) {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < MV_CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int x = 128 * c + 4 * lane + i;
                const float r = x < e ? y[0][4 * c + i] - lam * y[MAPS - 1][4 * c + i] : 0.f;
                y[0][4 * c + i] = r;
                ss = fmaf(r, r, ss);
            }
        ss = warp_sum(ss);
        const float f = 1.0f / sqrtf(ss / (float)e + eps);
#pragma unroll
        for (int c = 0; c < MV_CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int x = 128 * c + 4 * lane + i;
                if (x < e) st(o + x, (y[0][4 * c + i] * f) * factor);
            }
    } else {
#pragma unroll
        for (int c = 0; c < MV_CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int x = 128 * c + 4 * lane + i;
                if (x < e) st(o + x, y[0][4 * c + i]);
            }
    }
}

// ---------------------------------------------------------------------------
// One block per token.  The row [query latent (qr) | latent (r) | key part (dr) | gates (Hg)] is summed
// into shared memory; the two RMS norms follow (a block sum each); then the normed query latent goes out
// in the activation type, the normed latent and the turned key part go to the position's row of the
// cache ([page][64][r + dr]), and sigmoid(gate) goes out in float32.
//   pairing 0: (2i, 2i + 1) turn together; 1: (i, i + dr / 2).
template <typename T>
__global__ void __launch_bounds__(256)
latent_finish_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, int qr, int r, int dr, int Hg,
                     const float* __restrict__ q_w, const float* __restrict__ kv_w, float eps,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing, T* __restrict__ cq_out,
                     float* __restrict__ gate_out, T* __restrict__ rows, const int* __restrict__ page_table, int table_width,
                     const int* __restrict__ seq_of_token, const int* __restrict__ positions) {
    extern __shared__ float row[];
    __shared__ float red[40];
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    cos_t = fresh(cos_t);
    sin_t = fresh(sin_t);
    const int t = blockIdx.x, tid = threadIdx.x;
    const int W = qr + r + dr + Hg;
    for (int j = tid; j < W; j += blockDim.x) {
        float v = parts[(int64_t)t * W + j];
        for (int s = 1; s < splits; ++s) v += parts[s * split_stride + (int64_t)t * W + j];
        row[j] = v;
    }
    __syncthreads();
    float ss = 0.f;
    for (int j = tid; j < qr; j += blockDim.x) ss = fmaf(row[j], row[j], ss);
    ss = block_sum(ss, red);
    const float fq = 1.0f / sqrtf(ss / (float)qr + eps);
    for (int j = tid; j < qr; j += blockDim.x) st(cq_out + (int64_t)t * qr + j, (row[j] * fq) * q_w[j]);
    if (r > 0) {
        ss = 0.f;
        for (int j = tid; j < r; j += blockDim.x) ss = fmaf(row[qr + j], row[qr + j], ss);
        ss = block_sum(ss, red);
        if (rows) {
            const float fc = 1.0f / sqrtf(ss / (float)r + eps);
            const int pos = positions[t];
            const int pg = page_table[(int64_t)seq_of_token[t] * table_width + pos / kPage];
            T* dst = rows + ((int64_t)pg * kPage + pos % kPage) * (r + dr);
            for (int j = tid; j < r; j += blockDim.x) st(dst + j, (row[qr + j] * fc) * kv_w[j]);
            const int half = dr >> 1;
            const float* kr = row + qr + r;
            for (int i = tid; i < half; i += blockDim.x) {
                const int j0 = pairing == 0 ? 2 * i : i, j1 = pairing == 0 ? 2 * i + 1 : i + half;
                float u = kr[j0], v = kr[j1];
                if (cos_t) {
                    const float cs = cos_t[(int64_t)t * half + i], sn = sin_t[(int64_t)t * half + i];
                    const float ru = u * cs - v * sn, rv = v * cs + u * sn;
                    u = ru;
                    v = rv;
                }
                st(dst + r + j0, u);
                st(dst + r + j1, v);
            }
            if ((dr & 1) && tid == 0) st(dst + r + dr - 1, kr[dr - 1]);
        }
    }
    for (int j = tid; j < Hg; j += blockDim.x) gate_out[(int64_t)t * Hg + j] = 1.0f / (1.0f + expf(-row[qr + r + dr + j]));
}

// ---------------------------------------------------------------------------
// One block per (TT tokens, head).  The head's query [d | dr] of each token is summed into shared memory;
// thread j then makes element j of Wuk_h^T q for all TT tokens (a column of the head's d x r block of
// Wuk, read once for the TT tokens; sums over the d rows in index order), and the turned dr numbers follow it.
constexpr int LAT_TT = 8;

template <typename T>
__global__ void __launch_bounds__(256)
latent_absorb_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, const T* __restrict__ uk, int n, int H,
                     int d, int dr, int r, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing,
                     float* __restrict__ out) {
    extern __shared__ float qh[];                // [TT][d + dr]
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    cos_t = fresh(cos_t);
    sin_t = fresh(sin_t);
    const int t0 = blockIdx.x * LAT_TT, h = blockIdx.y, tid = threadIdx.x;
    const int dq = d + dr, W = H * dq, n_t = min(LAT_TT, n - t0);
    for (int idx = tid; idx < n_t * dq; idx += blockDim.x) {
        const int tt = idx / dq, x = idx - tt * dq;
        const int64_t at = (int64_t)(t0 + tt) * W + h * dq + x;
        float v = parts[at];
        for (int s = 1; s < splits; ++s) v += parts[s * split_stride + at];
        qh[tt * dq + x] = v;
    }
    for (int idx = tid + n_t * dq; idx < LAT_TT * dq; idx += blockDim.x) qh[idx] = 0.f;
    __syncthreads();
    const int half = dr >> 1;
    for (int idx = tid; idx < n_t * half; idx += blockDim.x) {
        const int tt = idx / half, i = idx - tt * half;
        const int j0 = pairing == 0 ? 2 * i : i, j1 = pairing == 0 ? 2 * i + 1 : i + half;
        float u = qh[tt * dq + d + j0], v = qh[tt * dq + d + j1];
        if (cos_t) {
            const float cs = cos_t[(int64_t)(t0 + tt) * half + i], sn = sin_t[(int64_t)(t0 + tt) * half + i];
            const float ru = u * cs - v * sn, rv = v * cs + u * sn;
            u = ru;
            v = rv;
        }
        float* o = out + ((int64_t)(t0 + tt) * H + h) * (r + dr) + r;
        o[j0] = u;
        o[j1] = v;
    }
    if ((dr & 1) && tid < n_t) out[((int64_t)(t0 + tid) * H + h) * (r + dr) + r + dr - 1] = qh[tid * dq + d + dr - 1];
    const T* w = uk + (int64_t)h * d * r;
    for (int j = tid; j < r; j += blockDim.x) {
        float acc[LAT_TT];
#pragma unroll
        for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = 0.f;
        for (int x = 0; x < d; ++x) {
            const float wv = ld(w + (int64_t)x * r + j);
#pragma unroll
            for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = fmaf(qh[tt * dq + x], wv, acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < LAT_TT; ++tt)
            if (tt < n_t) out[((int64_t)(t0 + tt) * H + h) * (r + dr) + j] = acc[tt];
    }
}

// One block per (TT tokens, head).  The head's weighted sums of latent rows (r numbers a token) wait in
// shared memory; a warp makes one output element for all TT tokens at a time: row x of the head's e x r
// block of Wuv, read once (lane l its elements l, l + 32, ...; the 32 sums by the butterfly), times the gate.
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_kernel(const float* __restrict__ y, const T* __restrict__ uv, const float* __restrict__ gate, int n, int H,
                     int e, int r, T* __restrict__ out) {
    extern __shared__ float ys[];                // [TT][r]
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    gate = fresh(gate);
    const int t0 = blockIdx.x * LAT_TT, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int n_t = min(LAT_TT, n - t0);
    for (int idx = tid; idx < LAT_TT * r; idx += blockDim.x) {
        const int tt = idx / r, j = idx - tt * r;
        ys[idx] = tt < n_t ? y[((int64_t)(t0 + tt) * H + h) * r + j] : 0.f;
    }
    __syncthreads();
    for (int x = warp; x < e; x += n_warps) {
        const T* w = uv + ((int64_t)h * e + x) * r;
        float acc[LAT_TT];
#pragma unroll
        for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = 0.f;
        for (int j = lane; j < r; j += 32) {
            const float wv = ld(w + j);
#pragma unroll
            for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = fmaf(ys[tt * r + j], wv, acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = warp_sum(acc[tt]);
        if (lane == 0) {
#pragma unroll
            for (int tt = 0; tt < LAT_TT; ++tt)
                if (tt < n_t) {
                    const float gt = gate ? gate[(int64_t)(t0 + tt) * H + h] : 1.f;
                    st(out + ((int64_t)(t0 + tt) * H + h) * e + x, acc[tt] * gt);
                }
        }
    }
}

// ---------------------------------------------------------------------------
template <typename T, typename TQ, typename TO, int MAPS>
int attn_multi(const void* q, const void* store, void* out, const int* seq_of_token, const int* positions,
               const int* page_table, int table_width, int n, int H, int G, int dm, int e, int64_t page_elems, int k_row,
               int64_t v_off, int v_row, float scale, int window, int keep_first, const float* sink, float lam, float eps,
               float factor, int few, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && G > 0 && H % G == 0 && dm > 0 && e > 0, "attn_multi: bad head counts or sizes");
    WICK_REQUIRE(e <= 128 * MV_CHUNKS, "attn_multi: a value size of %d is beyond %d", e, 128 * MV_CHUNKS);
    WICK_REQUIRE(window >= 0 && keep_first >= 0, "attn_multi: bad window");
    if (n == 0) return 0;
    // warps that share a token's keys: several where the step has few tokens, one where it has many
    const int warps = few ? 4 : 1;
    const int d_pad = (MAPS * dm + 3) & ~3, e_pad = (e + 127) / 128 * 128;
    const size_t smem = ((size_t)d_pad + 2 * MAPS * warps + (size_t)warps * MAPS * e_pad) * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "attn_multi: a head of %d numbers is beyond one block's shared memory", MAPS * dm);
    WICK_REQUIRE((int64_t)n * H <= 0x7fffffff, "attn_multi: too many (token, head) pairs");
    WICK_CUDA(launch(attn_multi_kernel<T, TQ, TO, MAPS>, dim3((unsigned)(n * H)), dim3(32 * warps), smem, s, (const TQ*)q, (const T*)store,
                     (TO*)out, seq_of_token, positions, page_table, table_width, H, G, dm, e, page_elems, k_row, v_off, v_row, scale,
                     window, keep_first, sink, lam, eps, factor));
    return check_launch("attn_multi");
}

template <typename T>
int latent_finish(const float* parts, int splits, int n, int qr, int r, int dr, int Hg, const float* q_w, const float* kv_w,
                  float eps, const float* cos_t, const float* sin_t, int pairing, void* cq_out, float* gate_out, void* rows,
                  const int* page_table, int table_width, const int* seq_of_token, const int* positions, cudaStream_t s) {
    WICK_REQUIRE(qr > 0 && r >= 0 && dr >= 0 && Hg >= 0 && splits >= 1, "latent_finish: bad sizes");
    WICK_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "latent_finish: the two angle tables come together");
    WICK_REQUIRE(!rows || (r > 0 && kv_w), "latent_finish: a cache row needs the latent and its norm weight");
    if (n == 0) return 0;
    const int W = qr + r + dr + Hg;
    const size_t smem = (size_t)W * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "latent_finish: a row of %d numbers is beyond one block's shared memory", W);
    WICK_CUDA(launch(latent_finish_kernel<T>, dim3(n), dim3(256), smem, s, parts, splits, (int64_t)n * W, qr, r, dr, Hg, q_w, kv_w, eps,
                     cos_t, sin_t, pairing, (T*)cq_out, gate_out, (T*)rows, page_table, table_width, seq_of_token, positions));
    return check_launch("latent_finish");
}

template <typename T>
int latent_absorb(const float* parts, int splits, const void* uk, int n, int H, int d, int dr, int r, const float* cos_t,
                  const float* sin_t, int pairing, float* out, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && d > 0 && dr >= 0 && r > 0 && splits >= 1, "latent_absorb: bad sizes");
    WICK_REQUIRE(H <= 65535, "latent_absorb: too many heads");
    if (n == 0) return 0;
    const size_t smem = (size_t)LAT_TT * (d + dr) * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "latent_absorb: a head of %d numbers is beyond one block's shared memory", d + dr);
    WICK_CUDA(launch(latent_absorb_kernel<T>, dim3(ceil_div(n, LAT_TT), H), dim3(256), smem, s, parts, splits,
                     (int64_t)n * H * (d + dr), (const T*)uk, n, H, d, dr, r, cos_t, sin_t, pairing, out));
    return check_launch("latent_absorb");
}

template <typename T>
int latent_expand(const float* y, const void* uv, const float* gate, int n, int H, int e, int r, void* out, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && e > 0 && r > 0 && H <= 65535, "latent_expand: bad sizes");
    if (n == 0) return 0;
    const size_t smem = (size_t)LAT_TT * r * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "latent_expand: a latent of %d numbers is beyond one block's shared memory", r);
    WICK_CUDA(launch(latent_expand_kernel<T>, dim3(ceil_div(n, LAT_TT), H), dim3(256), smem, s, y, (const T*)uv, gate, n, H, e, r, (T*)out));
    return check_launch("latent_expand");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

// q: [n, H, maps * dm] (maps = 2: the activation type; maps = 1: float32, a query carried into the rows' space);
// store: pages of page_elems elements; key row of (page, kv head g, place c): store + page * page_elems + (g * 64 + c) * k_row,
// value row: ... + v_off + (g * 64 + c) * v_row; out: [n, H, e] (maps = 2: activation type; maps = 1: float32).
#define WICK_ATTN_MULTI(NAME, T, TQ, TO, MAPS)                                                                                   \
    WICK_API int NAME(const void* q, const void* store, void* out, const int* seq_of_token, const int* positions,               \
                      const int* page_table, int table_width, int n, int H, int G, int dm, int e, int64_t page_elems, int k_row, \
                      int64_t v_off, int v_row, float scale, int window, int keep_first, const float* sink, float lam, float eps, \
                      float factor, int few, void* s) {                                                                          \
        return attn_multi<T, TQ, TO, MAPS>(q, store, out, seq_of_token, positions, page_table, table_width, n, H, G, dm, e,      \
                                           page_elems, k_row, v_off, v_row, scale, window, keep_first, sink, lam, eps, factor,   \
                                           few, (cudaStream_t)s);                                                                \
    }
WICK_ATTN_MULTI(wick_attn_multi2_bf16, bf16, bf16, bf16, 2)
WICK_ATTN_MULTI(wick_attn_multi2_f32, float, float, float, 2)
WICK_ATTN_MULTI(wick_attn_multi1_bf16, bf16, float, float, 1)
WICK_ATTN_MULTI(wick_attn_multi1_f32, float, float, float, 1)

#define WICK_LATENT(T, SUFFIX)                                                                                                   \
    WICK_API int wick_latent_finish_##SUFFIX(const float* parts, int splits, int n, int qr, int r, int dr, int Hg,              \
                                             const float* q_w, const float* kv_w, float eps, const float* cos_t,                \
                                             const float* sin_t, int pairing, void* cq_out, float* gate_out, void* rows,        \
                                             const int* page_table, int table_width, const int* seq_of_token,                   \
                                             const int* positions, void* s) {                                                   \
        return latent_finish<T>(parts, splits, n, qr, r, dr, Hg, q_w, kv_w, eps, cos_t, sin_t, pairing, cq_out, gate_out, rows,  \
                                page_table, table_width, seq_of_token, positions, (cudaStream_t)s);                              \
    }                                                                                                                            \
    WICK_API int wick_latent_absorb_##SUFFIX(const float* parts, int splits, const void* uk, int n, int H, int d, int dr, int r, \
                                             const float* cos_t, const float* sin_t, int pairing, float* out, void* s) {        \
        return latent_absorb<T>(parts, splits, uk, n, H, d, dr, r, cos_t, sin_t, pairing, out, (cudaStream_t)s);                 \
    }                                                                                                                            \
    WICK_API int wick_latent_expand_##SUFFIX(const float* y, const void* uv, const float* gate, int n, int H, int e, int r,     \
                                             void* out, void* s) {                                                              \
        return latent_expand<T>(y, uv, gate, n, H, e, r, out, (cudaStream_t)s);                                                  \
    }
WICK_LATENT(bf16, bf16)
WICK_LATENT(float, f32)
