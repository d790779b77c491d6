// Attention whose heads hold more than one score map, over paged storage described by
// strides, and the kernels around attention through a cached latent.
//
//   attend   : every new token over the cache (steps of few tokens: rows through shared memory, the keys in runs
//              over several blocks, then a merge).  A query head holds MAPS vectors of dm numbers;
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

constexpr int MV_MAX_CHUNKS = 4;                // value sizes up to 512: a lane holds 4 neighbours of every 128 (kernels are built for 1 and 4 such chunks)

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

// One block per (token, GROUP query heads, run of the visible keys); its warps share the run's keys, 32 at a
// time.  A block holds NQ = GROUP * MAPS query vectors of dm numbers ([head][map][dm], as they lie in memory); all
// of them score the same key rows (map a the a-th dm numbers of a row) and weigh the same value rows, so a row is
// read once for all of them.  In a tile, lane l scores key l of the tile for every vector (dot products in index
// order), the running maximum and sum of each follow, then every lane adds the tile's weighted value rows into its
// own elements of each vector's result.  The warps' partial results are folded in warp order, head gi by warp gi.
// With `partial` the fold's result goes there as a record (maximum, sum, two unused numbers, unnormalised values) per (token, head,
// map, run) for the merge kernel; without, the block holds all visible keys and finishes itself: the sink joins,
// the sums are divided, MAPS = 2 is combined (y_1 - lambda y_2, then the norm over the head's values).
template <int MAPS, int MV_CHUNKS>
__device__ __forceinline__ void finish_head(float (&y)[MAPS][4 * MV_CHUNKS], int lane, int e, float lam, float eps, float factor) {
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
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[0][c] = (y[0][c] * f) * factor;
    }
}

// The end of a block's work: the warps' running maxima, sums and unnormalised results (ms, accs: shared memory) are
// folded in warp order, head gi by warp gi; the result goes out as a record for the merge kernel (`partial`) or, where
// the block held all visible keys, is finished here (sink, division, two maps combined).
template <typename TO, int MAPS, int GROUP, int MV_CHUNKS>
__device__ __forceinline__ void fold_warps(float (&m)[MAPS * GROUP], float (&l)[MAPS * GROUP], float (&acc)[MAPS * GROUP][4 * MV_CHUNKS],
                                           float* ms, float* accs, TO* __restrict__ out, float* __restrict__ partial, int t, int h0,
                                           int H, int e, const float* __restrict__ sink, float lam, float eps, float factor) {
    constexpr int NQ = MAPS * GROUP;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int e_pad = (e + 127) / 128 * 128;
    if (lane == 0) {
#pragma unroll
        for (int a = 0; a < NQ; ++a) {
            ms[warp * NQ + a] = m[a];
            ms[(n_warps + warp) * NQ + a] = l[a];
        }
    }
#pragma unroll
    for (int a = 0; a < NQ; ++a)
#pragma unroll
        for (int c = 0; c < MV_CHUNKS; ++c)
            if (128 * c < e_pad)
#pragma unroll
                for (int i = 0; i < 4; ++i) accs[((int64_t)warp * NQ + a) * e_pad + 128 * c + 4 * lane + i] = acc[a][4 * c + i];
    __syncthreads();
    // warp gi folds head gi's maps over the block's warps; a lane holds its elements of the head's result
    for (int gi = warp; gi < GROUP; gi += n_warps) {
        const int h = h0 + gi;
        float y[MAPS][4 * MV_CHUNKS];
#pragma unroll
        for (int a = 0; a < MAPS; ++a) {
            const int qa = gi * MAPS + a;
            const bool with_sink = sink && !partial;
            float big = with_sink ? sink[h] : -INFINITY;
            for (int w = 0; w < n_warps; ++w) big = fmaxf(big, ms[w * NQ + qa]);
            float sum = with_sink ? expf(sink[h] - big) : 0.f;
#pragma unroll
            for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[a][c] = 0.f;
            for (int w = 0; w < n_warps; ++w) {
                const float mw = ms[w * NQ + qa];
                const float f = mw == -INFINITY ? 0.f : expf(mw - big);
                sum += ms[(n_warps + w) * NQ + qa] * f;
#pragma unroll
                for (int c = 0; c < MV_CHUNKS; ++c)
                    if (128 * c < e_pad)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            y[a][4 * c + i] = fmaf(accs[((int64_t)w * NQ + qa) * e_pad + 128 * c + 4 * lane + i], f, y[a][4 * c + i]);
            }
            if (partial) {                       // a record: maximum, sum, then the unnormalised values
                float* rec = partial + ((((int64_t)t * H + h) * MAPS + a) * gridDim.y + blockIdx.y) * (4 + e_pad);
                if (lane == 0) {
                    rec[0] = big;
                    rec[1] = sum;
                }
#pragma unroll
                for (int c = 0; c < MV_CHUNKS; ++c)
                    if (128 * c < e_pad) *reinterpret_cast<float4*>(rec + 4 + 128 * c + 4 * lane) =
                        make_float4(y[a][4 * c], y[a][4 * c + 1], y[a][4 * c + 2], y[a][4 * c + 3]);
            } else {
                const float inv = 1.0f / sum;    // (the block holds a visible key: the sum is positive)
#pragma unroll
                for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[a][c] *= inv;
            }
        }
        if (partial) continue;
        finish_head<MAPS, MV_CHUNKS>(y, lane, e, lam, eps, factor);
        TO* o = out + ((int64_t)t * H + h) * e;
#pragma unroll
        for (int c = 0; c < MV_CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int x = 128 * c + 4 * lane + i;
                if (x < e) st(o + x, y[0][4 * c + i]);
            }
    }
}

template <typename T, typename TQ, typename TO, int MAPS, int GROUP, int MV_CHUNKS>
__global__ void __launch_bounds__(256)
attn_multi_kernel(const TQ* __restrict__ q, const T* __restrict__ store, TO* __restrict__ out, float* __restrict__ partial,
                  const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                  const int* __restrict__ page_table, int table_width, int H, int G, int dm, int e, int64_t page_elems,
                  int k_row, int64_t v_off, int v_row, float scale, int window, int keep_first,
                  const float* __restrict__ sink, float lam, float eps, float factor) {
    constexpr int NQ = MAPS * GROUP;
    extern __shared__ __align__(16) float smem[];
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    store = fresh(store);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int groups = H / GROUP;
    const int t = blockIdx.x / groups, h0 = (blockIdx.x - t * groups) * GROUP;
    const int g = h0 / (H / G);                  // (a group's heads share a key/value head: GROUP divides H / G)
    const int pos = positions[t];
    const int* table = page_table + (int64_t)seq_of_token[t] * table_width;
    const int dq = NQ * dm, dq_pad = (dq + 3) & ~3, e_pad = (e + 127) / 128 * 128;
    float* qs = smem;                           // [NQ][dm]
    float* ms = qs + dq_pad;                    // [warps][NQ] maxima, then [warps][NQ] sums
    float* accs = ms + 2 * NQ * n_warps;        // [warps][NQ][e_pad]
    for (int x = threadIdx.x; x < dq; x += blockDim.x) qs[x] = ld(q + ((int64_t)t * H + h0) * (MAPS * dm) + x);
    __syncthreads();
    constexpr int VN = Vec16<T>::N;
    const bool base_ok = (((uintptr_t)store) & 15) == 0;
    const bool k_vec = base_ok && dm % VN == 0 && k_row % VN == 0 && page_elems % VN == 0;
    const bool v_vec = base_ok && e % 4 == 0 && v_row % 4 == 0 && page_elems % 4 == 0 && v_off % 4 == 0;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_kept = window > 0 ? min(keep_first, lo) : 0;
    const int total = n_kept + (pos - lo + 1);
    // this block's run of tiles
    const int tiles = (total + 31) >> 5, per_run = (tiles + (int)gridDim.y - 1) / (int)gridDim.y;
    const int v_begin = 32 * per_run * (int)blockIdx.y, v_end = min(total, 32 * per_run * ((int)blockIdx.y + 1));
    float m[NQ], l[NQ], acc[NQ][4 * MV_CHUNKS];
#pragma unroll
    for (int a = 0; a < NQ; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) acc[a][c] = 0.f;
    }
    for (int v0 = v_begin + 32 * warp; v0 < v_end; v0 += 32 * n_warps) {
        const int vi = v0 + lane;
        const bool valid = vi < v_end;
        float s[NQ], p[NQ];
#pragma unroll
        for (int a = 0; a < NQ; ++a) s[a] = 0.f;
        // where this lane's key row and value row lie (lanes beyond the run's end name its last key and weigh nothing)
        const int key = visible_key(min(vi, v_end - 1), n_kept, lo);
        const int64_t in_page = (int64_t)table[key / kPage] * page_elems, place = (int64_t)g * kPage + (key % kPage);
        const int64_t v_at = in_page + v_off + place * v_row;
        if (valid) {
            const T* kp = store + in_page + place * k_row;
#pragma unroll
            for (int a = 0; a < MAPS; ++a) {
                const T* ka = kp + a * dm;
                if (k_vec) {
                    for (int x = 0; x < dm; x += 4 * VN) {           // four loads of 16 bytes in flight
                        Vec16<T> kk[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (x + u * VN < dm) kk[u].load(ka + x + u * VN);
#pragma unroll
                        for (int gi = 0; gi < GROUP; ++gi) {
                            const float* qa = qs + (gi * MAPS + a) * dm + x;
                            float dot = s[gi * MAPS + a];
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (x + u * VN < dm) {
                                    // (the query's numbers four at a time: one trip to shared memory for four products)
#pragma unroll
                                    for (int i = 0; i < VN; i += 4) {
                                        const float4 q4 = *reinterpret_cast<const float4*>(qa + u * VN + i);
                                        dot = fmaf(q4.x, kk[u].v[i], dot);
                                        dot = fmaf(q4.y, kk[u].v[i + 1], dot);
                                        dot = fmaf(q4.z, kk[u].v[i + 2], dot);
                                        dot = fmaf(q4.w, kk[u].v[i + 3], dot);
                                    }
                                }
                            s[gi * MAPS + a] = dot;
                        }
                    }
                } else {
                    for (int x = 0; x < dm; ++x) {
                        const float kx = ld(ka + x);
#pragma unroll
                        for (int gi = 0; gi < GROUP; ++gi) s[gi * MAPS + a] = fmaf(qs[(gi * MAPS + a) * dm + x], kx, s[gi * MAPS + a]);
                    }
                }
            }
        }
#pragma unroll
        for (int a = 0; a < NQ; ++a) {
            s[a] = valid ? s[a] * scale : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max(s[a]));         // finite: the tile's first key is visible
            const float corr = expf(m[a] - m_new);                   // (m = -inf at first: 0)
            p[a] = valid ? expf(s[a] - m_new) : 0.f;
            l[a] = l[a] * corr + warp_sum(p[a]);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < 4 * MV_CHUNKS; ++c) acc[a][c] *= corr;
        }
        // the tile's value rows, each read by the whole warp; their places come from the lanes, so that the loads of
        // several rows are in flight together (a chain of look-ups and loads, row after row, is what a step of few
        // tokens would otherwise wait for)
        const int n_keys = min(32, v_end - v0);
#pragma unroll 4
        for (int jj = 0; jj < 32; ++jj) {
            if (jj >= n_keys) break;
            const T* vp = store + __shfl_sync(0xffffffffu, v_at, jj);
            float pj[NQ];
#pragma unroll
            for (int a = 0; a < NQ; ++a) pj[a] = __shfl_sync(0xffffffffu, p[a], jj);
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
                    for (int a = 0; a < NQ; ++a)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[a][4 * c + i] = fmaf(pj[a], vv[i], acc[a][4 * c + i]);
                }
            }
        }
    }
    fold_warps<TO, MAPS, GROUP, MV_CHUNKS>(m, l, acc, ms, accs, out, partial, t, h0, H, e, sink, lam, eps, factor);
}

// The form for steps of few tokens where rows can be copied 16 bytes at a time: one block per (token, GROUP heads, run
// of keys), as above, but the run's rows come through shared memory.  A tile of TK keys is copied there with cp.async
// (every copy of a tile in flight at once, the next tile's while this one is worked on), and a key row is then read by a
// WHOLE warp: lane l takes the row's 16-byte pieces l, l + 32, ... and its share of every query vector's dot product, the
// 32 shares are added by the butterfly.  A warp takes the keys w, w + 8, ... of a tile, four at a time: their scores, one
// step of the running maximum and sum, then their value rows (from the same tile in shared memory) into the lane's
// elements of every vector's result.  The warps' results are folded as above.
constexpr int TK = 32;                         // keys of a tile
constexpr int TW = 8;                          // warps of a block
constexpr int TS = 2;                          // tiles in shared memory: one worked on, one on its way (three were measured: slower, fewer blocks fit an SM)

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, typename TQ, typename TO, int MAPS, int GROUP, int MV_CHUNKS>
__global__ void __launch_bounds__(32 * TW)
attn_multi_tile_kernel(const TQ* __restrict__ q, const T* __restrict__ store, TO* __restrict__ out, float* __restrict__ partial,
                       const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                       const int* __restrict__ page_table, int table_width, int H, int G, int dm, int e, int64_t page_elems,
                       int k_row, int64_t v_off, int v_row, float scale, int window, int keep_first,
                       const float* __restrict__ sink, float lam, float eps, float factor) {
    constexpr int NQ = MAPS * GROUP;
    constexpr int VN = Vec16<T>::N;
    extern __shared__ __align__(16) float smem[];
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    store = fresh(store);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int groups = H / GROUP;
    const int t = blockIdx.x / groups, h0 = (blockIdx.x - t * groups) * GROUP;
    const int g = h0 / (H / G);
    const int pos = positions[t];
    const int* table = page_table + (int64_t)seq_of_token[t] * table_width;
    const int kd = MAPS * dm;                   // numbers of a key row
    const bool v_same = v_off == 0 && v_row == k_row;          // the value is the first e numbers of the key row
    const int row_elems = kd + (v_same ? 0 : e);                // a key's numbers in a tile: its key row, then its value row
    const int dq = NQ * dm, dq_pad = (dq + 3) & ~3, e_pad = (e + 127) / 128 * 128;
    float* qs = smem;                           // [NQ][dm]
    float* ms = qs + dq_pad;                    // [warps][NQ] maxima, then [warps][NQ] sums
    T* tiles = reinterpret_cast<T*>(ms + ((2 * NQ * TW + 3) & ~3));   // [TS][TK][row_elems]; afterwards the warps' results
    float* accs = reinterpret_cast<float*>(tiles);
    for (int x = tid; x < dq; x += blockDim.x) qs[x] = ld(q + ((int64_t)t * H + h0) * (MAPS * dm) + x);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_kept = window > 0 ? min(keep_first, lo) : 0;
    const int total = n_kept + (pos - lo + 1);
    const int n_tiles_all = (total + TK - 1) / TK, per_run = (n_tiles_all + (int)gridDim.y - 1) / (int)gridDim.y;
    const int v_begin = TK * per_run * (int)blockIdx.y, v_end = min(total, TK * per_run * ((int)blockIdx.y + 1));
    const int n_tiles = v_end > v_begin ? (v_end - v_begin + TK - 1) / TK : 0;
    const int kch = kd / VN, vch = v_same ? 0 : e / VN;                       // 16-byte pieces of a key's two rows

    // A key's rows are copied by 256 / TK neighbouring threads, which work out where the rows lie once a tile (the place of
    // every 16-byte piece on its own cost more instructions than the arithmetic on the tile).
    auto load_tile = [&](int it) {
        constexpr int TPK = 32 * TW / TK;       // threads that share a key
        T* dst = tiles + (int64_t)(it % TS) * TK * row_elems;
        const int v0 = v_begin + it * TK, n_keys = min(TK, v_end - v0);
        const int kk = tid / TPK, c0 = tid % TPK;
        if (kk < n_keys) {
            const int key = visible_key(v0 + kk, n_kept, lo);
            const int64_t in_page = (int64_t)table[key / kPage] * page_elems, place = (int64_t)g * kPage + (key % kPage);
            const T* ksrc = store + in_page + place * k_row;
            const T* vsrc = store + in_page + v_off + place * v_row;
            T* d = dst + (int64_t)kk * row_elems;
            for (int c = c0; c < kch; c += TPK) cp_async_16(d + c * VN, ksrc + c * VN);
            for (int c = c0; c < vch; c += TPK) cp_async_16(d + kd + c * VN, vsrc + c * VN);
        }
    };
#pragma unroll
    for (int it = 0; it < TS - 1; ++it) {       // (a group per tile, empty beyond the last, so that the waits below count alike)
        if (it < n_tiles) load_tile(it);
        cp_async_commit_group();
    }

    float m[NQ], l[NQ], acc[NQ][4 * MV_CHUNKS];
#pragma unroll
    for (int a = 0; a < NQ; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) acc[a][c] = 0.f;
    }
    constexpr int KW = TK / TW;                 // keys of a tile that one warp takes
    for (int it = 0; it < n_tiles; ++it) {
        if (it + TS - 1 < n_tiles) load_tile(it + TS - 1);       // (into the buffer that the barrier at the end of the last round freed)
        cp_async_commit_group();
        cp_async_wait_group<TS - 1>();
        __syncthreads();
        const T* tile = tiles + (int64_t)(it % TS) * TK * row_elems;
        const int n_keys = min(TK, v_end - (v_begin + it * TK));
        // scores of this warp's keys: a lane's share of every dot product, then the butterfly
        float s[KW][NQ];
#pragma unroll
        for (int j = 0; j < KW; ++j) {
            const int kk = warp + TW * j;
#pragma unroll
            for (int a = 0; a < NQ; ++a) s[j][a] = 0.f;
            if (kk < n_keys) {
                const T* kr = tile + (int64_t)kk * row_elems;
                for (int c = lane; c < kch; c += 32) {
                    Vec16<T> kv;
                    kv.load(kr + c * VN);
                    const int x0 = c * VN, a_of = MAPS == 1 ? 0 : x0 / dm, x_in = x0 - a_of * dm;
#pragma unroll
                    for (int gi = 0; gi < GROUP; ++gi)
#pragma unroll
                        for (int a = 0; a < MAPS; ++a) {
                            if (MAPS > 1 && a != a_of) continue;
                            const float* qa = qs + (gi * MAPS + a) * dm + x_in;
                            float dot = s[j][gi * MAPS + a];
#pragma unroll
                            for (int i = 0; i < VN; i += 4) {
                                const float4 q4 = *reinterpret_cast<const float4*>(qa + i);
                                dot = fmaf(q4.x, kv.v[i], dot);
                                dot = fmaf(q4.y, kv.v[i + 1], dot);
                                dot = fmaf(q4.z, kv.v[i + 2], dot);
                                dot = fmaf(q4.w, kv.v[i + 3], dot);
                            }
                            s[j][gi * MAPS + a] = dot;
                        }
                }
            }
#pragma unroll
            for (int a = 0; a < NQ; ++a) s[j][a] = kk < n_keys ? warp_sum(s[j][a]) * scale : -INFINITY;
        }
        // one step of the running maximum and sum for the warp's keys of this tile
        float p[KW][NQ];
#pragma unroll
        for (int a = 0; a < NQ; ++a) {
            float mx = m[a];
#pragma unroll
            for (int j = 0; j < KW; ++j) mx = fmaxf(mx, s[j][a]);
            if (mx == -INFINITY) {              // (the warp has seen no key yet)
#pragma unroll
                for (int j = 0; j < KW; ++j) p[j][a] = 0.f;
                continue;
            }
            const float corr = expf(m[a] - mx);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < KW; ++j) {
                p[j][a] = expf(s[j][a] - mx);   // (a key beyond the run's end: exp(-inf) = 0)
                sum += p[j][a];
            }
            l[a] = l[a] * corr + sum;
            m[a] = mx;
#pragma unroll
            for (int c = 0; c < 4 * MV_CHUNKS; ++c) acc[a][c] *= corr;
        }
        // the keys' value rows, from the tile
#pragma unroll
        for (int j = 0; j < KW; ++j) {
            const int kk = warp + TW * j;
            if (kk >= n_keys) continue;
            const T* vr = tile + (int64_t)kk * row_elems + (v_same ? 0 : kd);
#pragma unroll
            for (int c = 0; c < MV_CHUNKS; ++c) {
                const int x = 128 * c + 4 * lane;
                if (x < e) {
                    float vv[4];
                    mv_load4(vr + x, vv);
#pragma unroll
                    for (int a = 0; a < NQ; ++a)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[a][4 * c + i] = fmaf(p[j][a], vv[i], acc[a][4 * c + i]);
                }
            }
        }
        __syncthreads();                        // everyone is done with this buffer
    }
    fold_warps<TO, MAPS, GROUP, MV_CHUNKS>(m, l, acc, ms, accs, out, partial, t, h0, H, e, sink, lam, eps, factor);
}

// One warp per (token, head): the records of the runs of keys (a run that held no key has the maximum -inf) are
// folded in run order, map by map; the sink joins; the sums are divided; two maps are combined.
template <typename TO, int MAPS, int MV_CHUNKS>
__global__ void __launch_bounds__(128)
attn_multi_merge_kernel(const float* __restrict__ partial, TO* __restrict__ out, int n_heads_total, int H, int e, int runs,
                        const float* __restrict__ sink, float lam, float eps, float factor) {
    pdl_trigger();
    pdl_wait();
    partial = fresh(partial);
    const int lane = threadIdx.x & 31;
    const int th = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);      // token * H + head
    if (th >= n_heads_total) return;
    const int h = th % H, e_pad = (e + 127) / 128 * 128;
    float y[MAPS][4 * MV_CHUNKS];
#pragma unroll
    for (int a = 0; a < MAPS; ++a) {
        const float* recs = partial + ((int64_t)th * MAPS + a) * runs * (4 + e_pad);
        float big = sink ? sink[h] : -INFINITY;
        for (int r = 0; r < runs; ++r) big = fmaxf(big, recs[(int64_t)r * (4 + e_pad)]);
        float sum = sink ? expf(sink[h] - big) : 0.f;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[a][c] = 0.f;
        for (int r = 0; r < runs; ++r) {
            const float* rec = recs + (int64_t)r * (4 + e_pad);
            const float mr = rec[0];
            if (mr == -INFINITY) continue;
            const float f = expf(mr - big);
            sum += rec[1] * f;
#pragma unroll
            for (int c = 0; c < MV_CHUNKS; ++c)
                if (128 * c < e_pad) {
                    const float4 v = *reinterpret_cast<const float4*>(rec + 4 + 128 * c + 4 * lane);
                    y[a][4 * c] = fmaf(v.x, f, y[a][4 * c]);
                    y[a][4 * c + 1] = fmaf(v.y, f, y[a][4 * c + 1]);
                    y[a][4 * c + 2] = fmaf(v.z, f, y[a][4 * c + 2]);
                    y[a][4 * c + 3] = fmaf(v.w, f, y[a][4 * c + 3]);
                }
        }
        const float inv = 1.0f / sum;
#pragma unroll
        for (int c = 0; c < 4 * MV_CHUNKS; ++c) y[a][c] *= inv;
    }
    finish_head<MAPS, MV_CHUNKS>(y, lane, e, lam, eps, factor);
    TO* o = out + (int64_t)th * e;
#pragma unroll
    for (int c = 0; c < MV_CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int x = 128 * c + 4 * lane + i;
            if (x < e) st(o + x, y[0][4 * c + i]);
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
                     float* __restrict__ gate_out, T* __restrict__ rows, T* __restrict__ flat_c, T* __restrict__ flat_kr,
                     const int* __restrict__ page_table, int table_width,
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
            for (int j = tid; j < r; j += blockDim.x) {
                const float c = (row[qr + j] * fc) * kv_w[j];
                st(dst + j, c);
                if (flat_c) st(flat_c + (int64_t)t * r + j, c);
            }
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
                if (flat_kr) {
                    st(flat_kr + (int64_t)t * dr + j0, u);
                    st(flat_kr + (int64_t)t * dr + j1, v);
                }
            }
            if ((dr & 1) && tid == 0) {
                st(dst + r + dr - 1, kr[dr - 1]);
                if (flat_kr) st(flat_kr + (int64_t)t * dr + dr - 1, kr[dr - 1]);
            }
        }
    }
    for (int j = tid; j < Hg; j += blockDim.x) gate_out[(int64_t)t * Hg + j] = 1.0f / (1.0f + expf(-row[qr + r + dr + j]));
}

// ---------------------------------------------------------------------------
// The queries as they are, for kernels that score them against keys made from the latent: the partial sums are
// added up, the last dr numbers of every head [d | dr] are turned, and the row goes out in the activation type.
template <typename T>
__global__ void __launch_bounds__(256)
latent_query_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, int H, int d, int dr,
                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing, T* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    cos_t = fresh(cos_t);
    sin_t = fresh(sin_t);
    const int t = blockIdx.x, dq = d + dr, half = dr >> 1, per = d + half + (dr & 1);     // work items of a head: plain numbers, pairs
    const int64_t at = (int64_t)t * H * dq;
    auto sum = [&](int j) {
        float v = parts[at + j];
        for (int s = 1; s < splits; ++s) v += parts[s * split_stride + at + j];
        return v;
    };
    for (int idx = threadIdx.x; idx < H * per; idx += blockDim.x) {
        const int h = idx / per, i = idx - h * per;
        if (i < d) {
            st(out + at + h * dq + i, sum(h * dq + i));
        } else if (i - d < half) {
            const int p = i - d;
            const int j0 = h * dq + d + (pairing == 0 ? 2 * p : p), j1 = h * dq + d + (pairing == 0 ? 2 * p + 1 : p + half);
            float u = sum(j0), v = sum(j1);
            if (cos_t) {
                const float cs = cos_t[(int64_t)t * half + p], sn = sin_t[(int64_t)t * half + p];
                const float ru = u * cs - v * sn, rv = v * cs + u * sn;
                u = ru;
                v = rv;
            }
            st(out + at + j0, u);
            st(out + at + j1, v);
        } else {
            st(out + at + h * dq + dq - 1, sum(h * dq + dq - 1));
        }
    }
}

// ---------------------------------------------------------------------------
// One block per (TT tokens, head).  The head's query [d | dr] of each token is summed into shared memory;
// thread j then makes element j of Wuk_h^T q for all TT tokens (a column of the head's d x r block of
// Wuk, read once for the TT tokens; sums over the d rows in index order), and the turned dr numbers follow it.
constexpr int LAT_TT = 8;                       // (the kernels below spell out eight accumulators)

template <typename T>
__global__ void __launch_bounds__(256)
latent_absorb_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, const T* __restrict__ uk, int n, int H,
                     int d, int dr, int r, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairing,
                     float* __restrict__ out) {
    extern __shared__ __align__(16) float qh[];   // [d + dr][TT]: a number of all TT tokens side by side
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
        qh[x * LAT_TT + tt] = v;
    }
    for (int idx = tid; idx < (LAT_TT - n_t) * dq; idx += blockDim.x) qh[(idx % dq) * LAT_TT + n_t + idx / dq] = 0.f;
    __syncthreads();
    const int half = dr >> 1;
    for (int idx = tid; idx < (blockIdx.z == 0 ? n_t * half : 0); idx += blockDim.x) {
        const int tt = idx / half, i = idx - tt * half;
        const int j0 = pairing == 0 ? 2 * i : i, j1 = pairing == 0 ? 2 * i + 1 : i + half;
        float u = qh[(d + j0) * LAT_TT + tt], v = qh[(d + j1) * LAT_TT + tt];
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
    if ((dr & 1) && tid < n_t && blockIdx.z == 0) out[((int64_t)(t0 + tid) * H + h) * (r + dr) + r + dr - 1] = qh[(d + dr - 1) * LAT_TT + tid];
    const T* w = uk + (int64_t)h * d * r;
    for (int j = blockIdx.z * blockDim.x + tid; j < r; j += gridDim.z * blockDim.x) {      // (the blocks along z share the columns)
        float acc[LAT_TT];
#pragma unroll
        for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = 0.f;
#pragma unroll 8
        for (int x = 0; x < d; ++x) {                 // (eight rows' loads in flight: the kernel waits for them, not for arithmetic)
            const float wv = ld(w + (int64_t)x * r + j);
            const float4 qa = *reinterpret_cast<const float4*>(qh + x * LAT_TT), qb = *reinterpret_cast<const float4*>(qh + x * LAT_TT + 4);
            acc[0] = fmaf(qa.x, wv, acc[0]); acc[1] = fmaf(qa.y, wv, acc[1]); acc[2] = fmaf(qa.z, wv, acc[2]); acc[3] = fmaf(qa.w, wv, acc[3]);
            acc[4] = fmaf(qb.x, wv, acc[4]); acc[5] = fmaf(qb.y, wv, acc[5]); acc[6] = fmaf(qb.z, wv, acc[6]); acc[7] = fmaf(qb.w, wv, acc[7]);
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
    extern __shared__ __align__(16) float ys[];   // [r][TT]: a number of all TT tokens side by side
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    gate = fresh(gate);
    const int t0 = blockIdx.x * LAT_TT, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int n_t = min(LAT_TT, n - t0);
    for (int idx = tid; idx < LAT_TT * r; idx += blockDim.x) {
        const int tt = idx / r, j = idx - tt * r;
        ys[j * LAT_TT + tt] = tt < n_t ? y[((int64_t)(t0 + tt) * H + h) * r + j] : 0.f;
    }
    __syncthreads();
    for (int x = blockIdx.z * n_warps + warp; x < e; x += gridDim.z * n_warps) {             // (the blocks along z share the rows)
        const T* w = uv + ((int64_t)h * e + x) * r;
        float acc[LAT_TT];
#pragma unroll
        for (int tt = 0; tt < LAT_TT; ++tt) acc[tt] = 0.f;
#pragma unroll 4
        for (int j = lane; j < r; j += 32) {
            const float wv = ld(w + j);
            const float4 ya = *reinterpret_cast<const float4*>(ys + j * LAT_TT), yb = *reinterpret_cast<const float4*>(ys + j * LAT_TT + 4);
            acc[0] = fmaf(ya.x, wv, acc[0]); acc[1] = fmaf(ya.y, wv, acc[1]); acc[2] = fmaf(ya.z, wv, acc[2]); acc[3] = fmaf(ya.w, wv, acc[3]);
            acc[4] = fmaf(yb.x, wv, acc[4]); acc[5] = fmaf(yb.y, wv, acc[5]); acc[6] = fmaf(yb.z, wv, acc[6]); acc[7] = fmaf(yb.w, wv, acc[7]);
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
template <typename T, typename TQ, typename TO, int MAPS, int GROUP, int MV_CHUNKS>
int attn_multi_launch(const void* q, const void* store, void* out, float* partial, const int* seq_of_token, const int* positions,
                      const int* page_table, int table_width, int n, int H, int G, int dm, int e, int64_t page_elems, int k_row,
                      int64_t v_off, int v_row, float scale, int window, int keep_first, const float* sink, float lam, float eps,
                      float factor, int warps, int runs, cudaStream_t s) {
    constexpr int NQ = MAPS * GROUP;
    constexpr int VN = Vec16<T>::N;
    const int dq_pad = (NQ * dm + 3) & ~3, e_pad = (e + 127) / 128 * 128;
    // rows that can be copied 16 bytes at a time, in a step of few tokens: the form that reads them through shared memory
    const bool v_same = v_off == 0 && v_row == k_row;
    const bool copies = warps > 1 && ((uintptr_t)store & 15) == 0 && dm % VN == 0 && k_row % VN == 0 && page_elems % VN == 0 &&
                        e % VN == 0 && v_row % VN == 0 && v_off % VN == 0 && e % 4 == 0 && (MAPS * dm == k_row || !v_same);
    if (copies) {
        const size_t row_elems = (size_t)MAPS * dm + (v_same ? 0 : e);
        const size_t tile_bytes = (size_t)TS * TK * row_elems * sizeof(T), fold_bytes = (size_t)TW * NQ * e_pad * sizeof(float);
        const size_t smem = ((size_t)dq_pad + ((2 * NQ * TW + 3) & ~3)) * sizeof(float) + (tile_bytes > fold_bytes ? tile_bytes : fold_bytes);
        if (smem <= 200 * 1024) {
            static size_t raised = 48 * 1024;
            if (smem > raised) {
                WICK_CUDA(cudaFuncSetAttribute(attn_multi_tile_kernel<T, TQ, TO, MAPS, GROUP, MV_CHUNKS>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                raised = 200 * 1024;
            }
            WICK_CUDA(launch(attn_multi_tile_kernel<T, TQ, TO, MAPS, GROUP, MV_CHUNKS>, dim3((unsigned)(n * (H / GROUP)), runs), dim3(32 * TW),
                             smem, s, (const TQ*)q, (const T*)store, (TO*)out, partial, seq_of_token, positions, page_table, table_width,
                             H, G, dm, e, page_elems, k_row, v_off, v_row, scale, window, keep_first, sink, lam, eps, factor));
            if (int rc = check_launch("attn_multi_tile")) return rc;
            if (partial) {
                WICK_CUDA(launch(attn_multi_merge_kernel<TO, MAPS, MV_CHUNKS>, dim3(ceil_div((int64_t)n * H, 4)), dim3(128), 0, s,
                                 (const float*)partial, (TO*)out, n * H, H, e, runs, sink, lam, eps, factor));
                return check_launch("attn_multi_merge");
            }
            return 0;
        }
    }
    const size_t smem = ((size_t)dq_pad + 2 * NQ * warps + (size_t)warps * NQ * e_pad) * sizeof(float);
    WICK_REQUIRE(smem <= 160 * 1024, "attn_multi: heads of %d numbers are beyond one block's shared memory", NQ * dm);
    static size_t raised = 48 * 1024;
    if (smem > raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_multi_kernel<T, TQ, TO, MAPS, GROUP, MV_CHUNKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        raised = 160 * 1024;
    }
    WICK_CUDA(launch(attn_multi_kernel<T, TQ, TO, MAPS, GROUP, MV_CHUNKS>, dim3((unsigned)(n * (H / GROUP)), runs), dim3(32 * warps), smem, s,
                     (const TQ*)q, (const T*)store, (TO*)out, partial, seq_of_token, positions, page_table, table_width, H, G, dm, e,
                     page_elems, k_row, v_off, v_row, scale, window, keep_first, sink, lam, eps, factor));
    if (int rc = check_launch("attn_multi")) return rc;
    if (partial) {
        WICK_CUDA(launch(attn_multi_merge_kernel<TO, MAPS, MV_CHUNKS>, dim3(ceil_div((int64_t)n * H, 4)), dim3(128), 0, s, (const float*)partial,
                         (TO*)out, n * H, H, e, runs, sink, lam, eps, factor));
        return check_launch("attn_multi_merge");
    }
    return 0;
}

// few: the step has few tokens (one per sequence): eight warps share a block's keys, heads that read the same rows go
// through a block together (up to four), and the visible keys are cut into `runs` runs, a block each, whose records
// (`partial`: n * H * MAPS * runs * (4 + e rounded up to 128) floats, 16-byte aligned) a second kernel merges.
template <typename T, typename TQ, typename TO, int MAPS>
int attn_multi(const void* q, const void* store, void* out, float* partial, const int* seq_of_token, const int* positions,
               const int* page_table, int table_width, int n, int H, int G, int dm, int e, int64_t page_elems, int k_row,
               int64_t v_off, int v_row, float scale, int window, int keep_first, const float* sink, float lam, float eps,
               float factor, int few, int runs, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && G > 0 && H % G == 0 && dm > 0 && e > 0, "attn_multi: bad head counts or sizes");
    WICK_REQUIRE(e <= 128 * MV_MAX_CHUNKS, "attn_multi: a value size of %d is beyond %d", e, 128 * MV_MAX_CHUNKS);
    WICK_REQUIRE(window >= 0 && keep_first >= 0, "attn_multi: bad window");
    WICK_REQUIRE(runs >= 1 && runs <= 64 && (runs == 1 || partial), "attn_multi: %d runs of keys need a place for their records", runs);
    WICK_REQUIRE((int64_t)n * H <= 0x7fffffff, "attn_multi: too many (token, head) pairs");
    if (n == 0) return 0;
    if (runs == 1) partial = nullptr;
    const int per_kv = H / G;
    // (eight warps a block for a step of few tokens; four where the warps' results would fill a block's shared memory
    // and the step has blocks enough to fill the device twice without them)
#define WICK_AM(GROUP, CH)                                                                                                       \
    return attn_multi_launch<T, TQ, TO, MAPS, GROUP, CH>(q, store, out, partial, seq_of_token, positions, page_table, table_width, n, H, \
                                                         G, dm, e, page_elems, k_row, v_off, v_row, scale, window, keep_first, sink, \
                                                         lam, eps, factor, few ? (GROUP * CH > 4 && (int64_t)n * (H / GROUP) * runs > 2 * sm_count() ? 4 : 8) : 1, runs, s)
    if (e <= 128) {
        if (MAPS == 1 && few && per_kv % 4 == 0) WICK_AM(4, 1);
        if (MAPS == 1 && few && per_kv % 2 == 0) WICK_AM(2, 1);
        WICK_AM(1, 1);
    }
    if (MAPS == 1 && few && per_kv % 4 == 0) WICK_AM(4, 4);
    if (MAPS == 1 && few && per_kv % 2 == 0) WICK_AM(2, 4);
    WICK_AM(1, 4);
#undef WICK_AM
}

template <typename T>
int latent_finish(const float* parts, int splits, int n, int qr, int r, int dr, int Hg, const float* q_w, const float* kv_w,
                  float eps, const float* cos_t, const float* sin_t, int pairing, void* cq_out, float* gate_out, void* rows,
                  void* flat_c, void* flat_kr, const int* page_table, int table_width, const int* seq_of_token, const int* positions,
                  cudaStream_t s) {
    WICK_REQUIRE(qr > 0 && r >= 0 && dr >= 0 && Hg >= 0 && splits >= 1, "latent_finish: bad sizes");
    WICK_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "latent_finish: the two angle tables come together");
    WICK_REQUIRE(!rows || (r > 0 && kv_w), "latent_finish: a cache row needs the latent and its norm weight");
    if (n == 0) return 0;
    const int W = qr + r + dr + Hg;
    const size_t smem = (size_t)W * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "latent_finish: a row of %d numbers is beyond one block's shared memory", W);
    WICK_CUDA(launch(latent_finish_kernel<T>, dim3(n), dim3(256), smem, s, parts, splits, (int64_t)n * W, qr, r, dr, Hg, q_w, kv_w, eps,
                     cos_t, sin_t, pairing, (T*)cq_out, gate_out, (T*)rows, (T*)flat_c, (T*)flat_kr, page_table, table_width, seq_of_token,
                     positions));
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
    WICK_CUDA(launch(latent_absorb_kernel<T>, dim3(ceil_div(n, LAT_TT), H, min(64, ceil_div(r, 128))), dim3(128), smem, s, parts, splits,
                     (int64_t)n * H * (d + dr), (const T*)uk, n, H, d, dr, r, cos_t, sin_t, pairing, out));
    return check_launch("latent_absorb");
}

template <typename T>
int latent_query(const float* parts, int splits, int n, int H, int d, int dr, const float* cos_t, const float* sin_t, int pairing,
                 void* out, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && d > 0 && dr >= 0 && splits >= 1, "latent_query: bad sizes");
    if (n == 0) return 0;
    WICK_CUDA(launch(latent_query_kernel<T>, dim3(n), dim3(256), 0, s, parts, splits, (int64_t)n * H * (d + dr), H, d, dr, cos_t, sin_t,
                     pairing, (T*)out));
    return check_launch("latent_query");
}

template <typename T>
int latent_expand(const float* y, const void* uv, const float* gate, int n, int H, int e, int r, void* out, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && e > 0 && r > 0 && H <= 65535, "latent_expand: bad sizes");
    if (n == 0) return 0;
    const size_t smem = (size_t)LAT_TT * r * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "latent_expand: a latent of %d numbers is beyond one block's shared memory", r);
    WICK_CUDA(launch(latent_expand_kernel<T>, dim3(ceil_div(n, LAT_TT), H, min(64, ceil_div(e, 32))), dim3(256), smem, s, y, (const T*)uv, gate,
                     n, H, e, r, (T*)out));
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
                      float factor, int few, int runs, float* partial, void* s) {                                                \
        return attn_multi<T, TQ, TO, MAPS>(q, store, out, partial, seq_of_token, positions, page_table, table_width, n, H, G, dm, \
                                           e, page_elems, k_row, v_off, v_row, scale, window, keep_first, sink, lam, eps,        \
                                           factor, few, runs, (cudaStream_t)s);                                                  \
    }
WICK_ATTN_MULTI(wick_attn_multi2_bf16, bf16, bf16, bf16, 2)
WICK_ATTN_MULTI(wick_attn_multi2_f32, float, float, float, 2)
WICK_ATTN_MULTI(wick_attn_multi1_bf16, bf16, float, float, 1)
WICK_ATTN_MULTI(wick_attn_multi1_f32, float, float, float, 1)

#define WICK_LATENT(T, SUFFIX)                                                                                                   \
    WICK_API int wick_latent_finish_##SUFFIX(const float* parts, int splits, int n, int qr, int r, int dr, int Hg,              \
                                             const float* q_w, const float* kv_w, float eps, const float* cos_t,                \
                                             const float* sin_t, int pairing, void* cq_out, float* gate_out, void* rows,        \
                                             void* flat_c, void* flat_kr, const int* page_table, int table_width,               \
                                             const int* seq_of_token, const int* positions, void* s) {                          \
        return latent_finish<T>(parts, splits, n, qr, r, dr, Hg, q_w, kv_w, eps, cos_t, sin_t, pairing, cq_out, gate_out, rows,  \
                                flat_c, flat_kr, page_table, table_width, seq_of_token, positions, (cudaStream_t)s);             \
    }                                                                                                                            \
    WICK_API int wick_latent_absorb_##SUFFIX(const float* parts, int splits, const void* uk, int n, int H, int d, int dr, int r, \
                                             const float* cos_t, const float* sin_t, int pairing, float* out, void* s) {        \
        return latent_absorb<T>(parts, splits, uk, n, H, d, dr, r, cos_t, sin_t, pairing, out, (cudaStream_t)s);                 \
    }                                                                                                                            \
    WICK_API int wick_latent_query_##SUFFIX(const float* parts, int splits, int n, int H, int d, int dr, const float* cos_t,     \
                                            const float* sin_t, int pairing, void* out, void* s) {                               \
        return latent_query<T>(parts, splits, n, H, d, dr, cos_t, sin_t, pairing, out, (cudaStream_t)s);                         \
    }                                                                                                                            \
    WICK_API int wick_latent_expand_##SUFFIX(const float* y, const void* uv, const float* gate, int n, int H, int e, int r,     \
                                             void* out, void* s) {                                                              \
        return latent_expand<T>(y, uv, gate, n, H, e, r, out, (cudaStream_t)s);                                                  \
    }
WICK_LATENT(bf16, bf16)
WICK_LATENT(float, f32)
