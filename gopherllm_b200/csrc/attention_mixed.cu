// Softmax attention over the paged cache whose heads' weights are mixed before they meet the
// values, with keys and values of different sizes; 32-bit arithmetic, any sizes, both element types.
//
// With weights p_g(i, j) = softmax_j(q_g(i) . k(j)) of query head g, head h of the mixer applies
//     w_h(i, j) = sum_g M[h, g] p_g(i, j)
// to the values of its own key/value head c(h).  The sum over j is linear, so
//     out_h(i) = sum_g M[h, g] * A[g, c(h)](i),     A[g, c](i) = sum_j p_g(i, j) v_c(j):
// the first kernel computes A for every pair (query head, value head) with a running maximum and
// sum (a pair's scores come from the query head's own key head), the second mixes.  Without a table
// the pairs are (g, c(g)) alone and the second kernel only converts.  A query at position p sees keys
// lo..p, lo = 0 or p-window+1.
//
// A score may be shaped before the softmax: s = (q . k) * score_scale; with softcap > 0,
// s <- softcap * tanh(s / softcap); with a slope per query head, s <- s - slope_h * (p - j) for the
// key at position j (a penalty that grows with the distance).  A head may have a sink: a learned score that
// joins the denominator of its softmax once, unscaled, with no key and no value.
#include "common.cuh"

struct MixedAttnArgs {
    const void* q;            // [T, nH*hd] activation type, already scaled
    float* pairs;             // [T, nH, nVal, vd] 32-bit; nVal = nKV with a table, 1 without
    void* out;                // [T, nH*vd] activation type
    const void* k_cache;      // [pages, nKV, GL_PAGE, hd] cache type
    const void* v_cache;      // [pages, nKV (nVH), GL_PAGE, vd] cache type
    const float* mix;         // [nH, nH] or null
    const int* seq_qstart;
    const int* seq_qlen;
    const int* seq_ctx;
    const int* pages;         // [B, max_pages]
    int T, B, nH, nKV, hd, vd, max_pages, window, max_qlen;
    int n_pages;
    // one token a sequence, the context cut into ``splits`` ranges of pages, a block each:
    float* parts;             // [B, nH, nVal, splits, vd] sums not yet divided
    float* ml;                // [B, nH, splits, 2] each range's maximum and sum
    int splits, pages_per_split;
    float score_scale;        // multiplies q . k
    float softcap;            // > 0: scores are capped smoothly at +-softcap
    const float* slopes;      // [nH] or null: head h's penalty per position of distance
    const float* sinks;       // [nH] or null: e^(sinks[h]) joins the softmax's denominator of head h (no key, no value)
    int nVH;                  // heads of the value cache where they are more than the key heads (a multiple of nKV; 0: nKV):
                              // without a table, query head g then takes the values of head g / (nH / nVH)
    int vs;                   // numbers between two positions' values of a head (0: vd).  A cache whose values are the
                              // first vd columns of its key rows is read with v_cache = k_cache and vs = hd
};

__host__ __device__ __forceinline__ int am_value_stride(const MixedAttnArgs& a) { return a.vs > 0 ? a.vs : a.vd; }

__host__ __device__ __forceinline__ int am_value_heads(const MixedAttnArgs& a) { return a.nVH > 0 ? a.nVH : a.nKV; }

// What a sink does to a finished softmax with maximum m and sum l (of e^(s - m)): the factor on the weighted
// values' sum, 1 / (l + e^(sink - m)), taken against the larger of m and the sink so that nothing overflows.
__device__ __forceinline__ float am_finish(float m, float l, const float* sinks, int h) {
    if (!sinks) return l > 0.f ? 1.0f / l : 0.f;
    const float sink = sinks[h];
    const float top = fmaxf(m, sink);
    const float scale = m > -INFINITY ? expf(m - top) : 0.f;
    return scale / (l * scale + expf(sink - top));
}

// the shaped score of query head h at position p and the key at position j
__device__ __forceinline__ float am_shape(float dot, const MixedAttnArgs& a, float slope, int p, int j) {
    float s = dot * a.score_scale;
    if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
    return s - slope * (float)(p - j);
}

#define AM_ROWS 8

// Prompts: one warp owns one query row of one pair; the warps of a block are consecutive tokens of a
// sequence and share the key and value tiles staged in shared memory: a page at a time, or (``stage_rows`` 32, for
// key rows too long for a whole page of them to fit) half a page at a time.
template <typename TA, typename TC, int NACC>
__global__ void __launch_bounds__(AM_ROWS * 32)
attn_pairs_kernel(MixedAttnArgs a, int stage_rows) {
    extern __shared__ float smem[];
    gl_grid_wait();
    const int hd = a.hd, vd = a.vd, ks = hd + 1;
    float* Ks = smem;                       // [stage_rows][hd+1]
    float* Vs = Ks + stage_rows * ks;       // [stage_rows][vd]
    float* Qs = Vs + stage_rows * vd;       // [AM_ROWS][hd]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z;
    const int nVal = a.mix ? a.nKV : 1;
    const int g = blockIdx.y / nVal;                              // query head
    const int kh = g / (a.nH / a.nKV);                            // its key head
    const int nvh = am_value_heads(a);
    const int vh = a.mix ? blockIdx.y - g * nVal : g / (a.nH / nvh);      // the pair's value head
    const int qlen = a.seq_qlen[b];
    const int row0 = blockIdx.x * AM_ROWS;
    if (row0 >= qlen) return;
    const int ctx = a.seq_ctx[b];
    const int total = ctx + qlen;
    const int idx = row0 + warp;
    const bool live = idx < qlen;
    const int p = ctx + idx;
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int rows_here = min(AM_ROWS, qlen - row0);
    const int p_first = ctx + row0, p_last = ctx + row0 + rows_here - 1;
    const int lo_cta = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;

    float* qv = Qs + warp * hd;
    const float slope = a.slopes ? a.slopes[g] : 0.f;
    if (live) {
        const TA* qsrc = (const TA*)a.q + ((size_t)(a.seq_qstart[b] + idx) * a.nH + g) * hd;
        for (int d = lane; d < hd; d += 32) qv[d] = gl_load(qsrc + d);
    }
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int* pg = a.pages + (size_t)b * a.max_pages;
    for (int page_i = lo_cta / GL_PAGE; page_i <= p_last / GL_PAGE; ++page_i) {
        const int page = gl_checked(pg[gl_checked(page_i, a.max_pages, GL_BAD_POSITION)], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
        const TC* kp = (const TC*)a.k_cache + ((size_t)page * a.nKV + kh) * GL_PAGE * hd;
        const int vs = am_value_stride(a);
        const TC* vp = (const TC*)a.v_cache + ((size_t)page * nvh + vh) * GL_PAGE * vs;
        for (int row0s = 0; row0s < GL_PAGE; row0s += stage_rows) {
        const int j0 = page_i * GL_PAGE + row0s;
        __syncthreads();
        for (int e = threadIdx.x; e < stage_rows * hd; e += blockDim.x) {
            const int r = e / hd, d = e - r * hd;
            Ks[r * ks + d] = j0 + r < total ? gl_load(kp + (size_t)row0s * hd + e) : 0.f;      // rows past the sequence were never written
        }
        for (int e = threadIdx.x; e < stage_rows * vd; e += blockDim.x) {
            const int r = e / vd;
            Vs[e] = j0 + r < total ? gl_load(vp + (size_t)(row0s + r) * vs + (e - r * vd)) : 0.f;
        }
        __syncthreads();
        if (!live) continue;
#pragma unroll 1
        for (int half = 0; half < stage_rows / 32; ++half) {
            const int jj = half * 32 + lane, j = j0 + jj;
            const bool ok = j >= lo && j <= p;
            float s = -INFINITY;
            if (ok) {
                const float* kr = Ks + jj * ks;
                float d0 = 0.f;
                for (int d = 0; d < hd; ++d) d0 = fmaf(qv[d], kr[d], d0);
                s = am_shape(d0, a, slope, p, j);
            }
            const float m_new = fmaxf(m, gl_warp_max(s));
            if (m_new == -INFINITY) continue;
            const float pj = ok ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);
            l = l * corr + gl_warp_sum(pj);
            m = m_new;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] *= corr;
            const float* vr = Vs + half * 32 * vd;
            for (int k = 0; k < 32; ++k) {
                const float pk = __shfl_sync(0xffffffffu, pj, k);
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int d = lane + 32 * i;
                    if (d < vd) acc[i] = fmaf(pk, vr[k * vd + d], acc[i]);
                }
            }
        }
        }
    }
    if (!live) return;
    const float inv = am_finish(m, l, a.sinks, g);
    float* o = a.pairs + (((size_t)(a.seq_qstart[b] + idx) * a.nH + g) * nVal + (a.mix ? vh : 0)) * vd;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) o[d] = acc[i] * inv;
    }
}

// One token a sequence: a block owns one pair of one sequence, its warps take the pages of the
// context in turn straight from the cache (a lane a key for the scores, a lane a column for the
// values) and their partial results are merged in shared memory in warp order.
#define AM_DWARPS 8

template <typename TA, typename TC, int NACC>
__global__ void __launch_bounds__(AM_DWARPS * 32)
attn_pairs_decode_kernel(MixedAttnArgs a) {
    extern __shared__ float smem[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int hd = a.hd, vd = a.vd;
    float* qv = smem;                                   // [hd]
    float* part = qv + hd;                              // [AM_DWARPS][vd + 2]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    const int nVal = a.mix ? a.nKV : 1;
    const int g = blockIdx.x / nVal;
    const int kh = g / (a.nH / a.nKV);
    const int nvh = am_value_heads(a);
    const int vh = a.mix ? blockIdx.x - g * nVal : g / (a.nH / nvh);
    const int p = a.seq_ctx[b];                         // the token's position; keys lo..p
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int row = a.seq_qstart[b];
    const TA* qsrc = (const TA*)a.q + ((size_t)row * a.nH + g) * hd;
    const float slope = a.slopes ? a.slopes[g] : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) qv[d] = gl_load(qsrc + d);
    __syncthreads();
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int* pg = a.pages + (size_t)b * a.max_pages;
    for (int page_i = lo / GL_PAGE + warp; page_i <= p / GL_PAGE; page_i += AM_DWARPS) {
        const int page = gl_checked(pg[gl_checked(page_i, a.max_pages, GL_BAD_POSITION)], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
        const TC* kp = (const TC*)a.k_cache + ((size_t)page * a.nKV + kh) * GL_PAGE * hd;
        const int vs = am_value_stride(a);
        const TC* vp = (const TC*)a.v_cache + ((size_t)page * nvh + vh) * GL_PAGE * vs;
        const int j0 = page_i * GL_PAGE;
#pragma unroll 1
        for (int half = 0; half < GL_PAGE / 32; ++half) {
            const int jj = half * 32 + lane, j = j0 + jj;
            const bool ok = j >= lo && j <= p;
            float s = -INFINITY;
            if (ok) {
                const TC* kr = kp + (size_t)jj * hd;
                float d0 = 0.f;
                for (int d = 0; d < hd; ++d) d0 = fmaf(qv[d], gl_load(kr + d), d0);
                s = am_shape(d0, a, slope, p, j);
            }
            const float m_new = fmaxf(m, gl_warp_max(s));
            if (m_new == -INFINITY) continue;
            const float pj = ok ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);
            l = l * corr + gl_warp_sum(pj);
            m = m_new;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] *= corr;
            const TC* vr = vp + (size_t)half * 32 * vs;
            // keys past p were never written, keys before lo may lie in a page that was given back
            const int kmin = max(0, lo - (j0 + half * 32)), kmax = min(32, p - (j0 + half * 32) + 1);
            for (int k = kmin; k < kmax; ++k) {
                const float pk = __shfl_sync(0xffffffffu, pj, k);
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int d = lane + 32 * i;
                    if (d < vd) acc[i] = fmaf(pk, gl_load(vr + (size_t)k * vs + d), acc[i]);
                }
            }
        }
    }
    float* mine = part + warp * (vd + 2);
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) mine[d] = acc[i];
    }
    if (lane == 0) { mine[vd] = m; mine[vd + 1] = l; }
    __syncthreads();
    float mm = -INFINITY;
    for (int w = 0; w < AM_DWARPS; ++w) mm = fmaxf(mm, part[w * (vd + 2) + vd]);
    float ll = 0.f;
    for (int w = 0; w < AM_DWARPS; ++w) {
        const float mw = part[w * (vd + 2) + vd];
        if (mw > -INFINITY) ll += part[w * (vd + 2) + vd + 1] * expf(mw - mm);
    }
    const float inv = am_finish(mm, ll, a.sinks, g);
    float* o = a.pairs + (((size_t)row * a.nH + g) * nVal + (a.mix ? vh : 0)) * vd;
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < AM_DWARPS; ++w) {
            const float mw = part[w * (vd + 2) + vd];
            if (mw > -INFINITY) s = fmaf(part[w * (vd + 2) + d], expf(mw - mm), s);
        }
        o[d] = s * inv;
    }
}

// One token a sequence, few heads a group: a block owns one key head of one sequence, that is the query
// heads that share it (up to eight; where more share a key head, as when every head reads one wide key row, a
// block owns a run of eight of them), and every value head their weights are applied to.  A page of keys is read once
// for all of the group's query heads (a thread a (head, key) score), the softmax of a head is kept by one
// warp, and each warp accumulates one value head for all of the group's query heads, so a page of values
// is read once per key head and not once per pair.
#define AM_GTHREADS 256

__device__ __forceinline__ float am_dot(const float* q, const __nv_bfloat16* k, int hd) {
    float acc = 0.f;
    if ((hd & 7) == 0) {
        for (int d = 0; d < hd; d += 8) {
            const uint4 raw = *(const uint4*)(k + d);
            const __nv_bfloat162* p2 = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(p2[e]);
                acc = fmaf(q[d + 2 * e], f.x, acc);
                acc = fmaf(q[d + 2 * e + 1], f.y, acc);
            }
        }
    } else {
        for (int d = 0; d < hd; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
    }
    return acc;
}
__device__ __forceinline__ float am_dot(const float* q, const float* k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; ++d) acc = fmaf(q[d], k[d], acc);
    return acc;
}

template <typename TA, typename TC, int NACC, int GQ>
__global__ void __launch_bounds__(AM_GTHREADS)
attn_group_decode_kernel(MixedAttnArgs a) {
    extern __shared__ float smem[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int hd = a.hd, vd = a.vd;
    const int group = a.nH / a.nKV;                     // query heads of a key head
    const int gq = group < GQ ? group : GQ;             // of this block (<= GQ); group is a multiple of it
    const int chunks = group / gq;
    float* qv = smem;                                   // [gq][hd]
    float* sc = qv + gq * hd;                           // [gq][GL_PAGE] scores, then weights
    float* corr = sc + gq * GL_PAGE;                    // [gq] rescaling of this page, then 1 / sum
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y, kh = blockIdx.x / chunks, split = blockIdx.z;
    const int head0 = kh * group + (blockIdx.x - kh * chunks) * gq;      // this block's first query head
    const int nVal = a.mix ? a.nKV : 1;
    const int p = a.seq_ctx[b];
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int row = a.seq_qstart[b];
    const int page_first = lo / GL_PAGE + split * a.pages_per_split;
    const int page_last = min(p / GL_PAGE, page_first + a.pages_per_split - 1);      // may lie before page_first: nothing to do
    const TA* qsrc = (const TA*)a.q + ((size_t)row * a.nH + (size_t)head0) * hd;
    for (int i = threadIdx.x; i < gq * hd; i += AM_GTHREADS) qv[i] = gl_load(qsrc + i);
    // this warp's value head: with a table every value head meets every query head; without one the key head's
    // query heads fall into as many equal runs as it has value heads, a warp a run
    const int nvh = am_value_heads(a);
    const int share = a.nH / nvh;                       // query heads that share a value head
    const int per = share < gq ? share : gq;            // ... among this block's
    const int runs = a.mix ? 1 : gq / per;              // value heads of this block
    const int vh = a.mix ? warp : head0 / share + warp;
    const bool has_values = a.mix ? warp < a.nKV : warp < runs;
    float acc[GQ][NACC];
#pragma unroll
    for (int g = 0; g < GQ; ++g)
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[g][i] = 0.f;
    float m = -INFINITY, l = 0.f;                       // warp g < gq keeps head g's running maximum and sum
    const int* pg = a.pages + (size_t)b * a.max_pages;
    for (int page_i = page_first; page_i <= page_last; ++page_i) {
        const int page = gl_checked(pg[gl_checked(page_i, a.max_pages, GL_BAD_POSITION)], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
        const TC* kp = (const TC*)a.k_cache + ((size_t)page * a.nKV + kh) * GL_PAGE * hd;
        const int j0 = page_i * GL_PAGE;
        __syncthreads();                                // the page before is used up (and q is in place)
        for (int item = threadIdx.x; item < gq * GL_PAGE; item += AM_GTHREADS) {
            const int g = item / GL_PAGE, key = item - g * GL_PAGE;
            const int j = j0 + key;
            sc[item] = (j >= lo && j <= p)
                ? am_shape(am_dot(qv + g * hd, kp + (size_t)key * hd, hd), a, a.slopes ? a.slopes[head0 + g] : 0.f, p, j)
                : -INFINITY;
        }
        __syncthreads();
        if (warp < gq) {
            const float s0 = sc[warp * GL_PAGE + lane], s1 = sc[warp * GL_PAGE + 32 + lane];
            const float m_new = fmaxf(m, gl_warp_max(fmaxf(s0, s1)));      // the page holds position lo or later: finite
            const float p0 = s0 > -INFINITY ? expf(s0 - m_new) : 0.f, p1 = s1 > -INFINITY ? expf(s1 - m_new) : 0.f;
            const float c = expf(m - m_new);                                 // m = -inf gives 0
            l = l * c + gl_warp_sum(p0 + p1);
            m = m_new;
            sc[warp * GL_PAGE + lane] = p0;
            sc[warp * GL_PAGE + 32 + lane] = p1;
            if (lane == 0) corr[warp] = c;
        }
        __syncthreads();
        if (has_values) {
            const int vs = am_value_stride(a);
            const TC* vp = (const TC*)a.v_cache + ((size_t)page * nvh + vh) * GL_PAGE * vs;
#pragma unroll
            for (int g = 0; g < GQ; ++g) {
                if (g < gq) {
                    const float c = corr[g];
#pragma unroll
                    for (int i = 0; i < NACC; ++i) acc[g][i] *= c;
                }
            }
            const int kmin = max(0, lo - j0), kmax = min(GL_PAGE, p - j0 + 1);   // written keys inside the window
            // sixteen keys' values are asked for before the first is used: one after the other, every key
            // would cost a trip to memory
            constexpr int KB = NACC <= 2 ? 16 : 8;
            for (int k0 = 0; k0 < GL_PAGE; k0 += KB) {
                if (k0 + KB <= kmin || k0 >= kmax) continue;
                float v[KB][NACC];
#pragma unroll
                for (int kk = 0; kk < KB; ++kk) {
                    const bool ok = k0 + kk >= kmin && k0 + kk < kmax;
#pragma unroll
                    for (int i = 0; i < NACC; ++i) {
                        const int d = lane + 32 * i;
                        v[kk][i] = (ok && d < vd) ? gl_load(vp + (size_t)(k0 + kk) * vs + d) : 0.f;
                    }
                }
#pragma unroll
                for (int kk = 0; kk < KB; ++kk) {
#pragma unroll
                    for (int g = 0; g < GQ; ++g) {
                        if (g < gq && (a.mix || g / per == warp)) {
                            const float pk = sc[g * GL_PAGE + k0 + kk];
#pragma unroll
                            for (int i = 0; i < NACC; ++i) acc[g][i] = fmaf(pk, v[kk][i], acc[g][i]);
                        }
                    }
                }
            }
        }
    }
    // the range's sums as they are, with its maximum and sum: the mixing kernel puts the ranges together
    if (warp < gq && lane == 0) {
        float* dst = a.ml + (((size_t)b * a.nH + (size_t)head0 + warp) * a.splits + split) * 2;
        dst[0] = m;
        dst[1] = l;
    }
    if (has_values) {
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
            if (g < gq && (a.mix || g / per == warp)) {
                float* o = a.parts + ((((size_t)b * a.nH + (size_t)head0 + g) * nVal + (a.mix ? vh : 0)) * a.splits + split) * vd;
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int d = lane + 32 * i;
                    if (d < vd) o[d] = acc[g][i];
                }
            }
        }
    }
}

// out[b, h, :] = sum_g M[h, g] * (sum_s parts[b, g, c(h), s, :] e^(m_gs - m_g)) / (sum_s l_gs e^(m_gs - m_g))
template <typename TA>
__global__ void __launch_bounds__(128)
head_mix_split_kernel(MixedAttnArgs a) {
    extern __shared__ float coef[];                     // [heads taken][splits]: M[h, g] e^(m_gs - m_g) / sum_g
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.y, h = blockIdx.x;
    const int nVal = a.mix ? a.nKV : 1;
    const int c = a.mix ? h / (a.nH / a.nKV) : 0;
    const int row = a.seq_qstart[b];
    const int g0 = a.mix ? 0 : h, ng = a.mix ? a.nH : 1;
    for (int gi = threadIdx.x; gi < ng; gi += blockDim.x) {
        const int g = g0 + gi;
        const float* ml = a.ml + ((size_t)b * a.nH + g) * a.splits * 2;
        float mm = -INFINITY;
        for (int s = 0; s < a.splits; ++s) mm = fmaxf(mm, ml[2 * s]);
        float den = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float e = ml[2 * s] > -INFINITY ? expf(ml[2 * s] - mm) : 0.f;
            coef[gi * a.splits + s] = e;
            den = fmaf(ml[2 * s + 1], e, den);
        }
        const float w = (a.mix ? a.mix[h * a.nH + g] : 1.0f) * am_finish(mm, den, a.sinks, g);
        for (int s = 0; s < a.splits; ++s) coef[gi * a.splits + s] *= w;
    }
    __syncthreads();
    const int terms = ng * a.splits;
    for (int d = threadIdx.x; d < a.vd; d += blockDim.x) {
        float y = 0.f;
#pragma unroll 8
        for (int i = 0; i < terms; ++i) {
            const int gi = i / a.splits, s = i - gi * a.splits;
            y = fmaf(coef[i], a.parts[((((size_t)b * a.nH + g0 + gi) * nVal + c) * a.splits + s) * a.vd + d], y);
        }
        gl_store((TA*)a.out + ((size_t)row * a.nH + h) * a.vd + d, y);
    }
}

template <typename TA, typename TC, int NACC>
static int launch_group_decode(const MixedAttnArgs& a, cudaStream_t stream) {
    const int group = a.nH / a.nKV, gq = group < 8 ? group : 8;
    const size_t smem = ((size_t)gq * a.hd + (size_t)gq * GL_PAGE + gq) * sizeof(float);
    const dim3 grid(a.nKV * (group / gq), a.B, a.splits);
    if (gq <= 1) return gl_launch(attn_group_decode_kernel<TA, TC, NACC, 1>, grid, dim3(AM_GTHREADS), smem, stream, 1, a);
    if (gq <= 2) return gl_launch(attn_group_decode_kernel<TA, TC, NACC, 2>, grid, dim3(AM_GTHREADS), smem, stream, 1, a);
    if (gq <= 4) return gl_launch(attn_group_decode_kernel<TA, TC, NACC, 4>, grid, dim3(AM_GTHREADS), smem, stream, 1, a);
    return gl_launch(attn_group_decode_kernel<TA, TC, NACC, 8>, grid, dim3(AM_GTHREADS), smem, stream, 1, a);
}

// out[t, h, :] = sum_g M[h, g] pairs[t, g, c(h), :]   (without a table: pairs[t, h, 0, :])
template <typename TA>
__global__ void __launch_bounds__(256)
head_mix_kernel(MixedAttnArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n = (long long)a.T * a.nH * a.vd;
    if (i >= n) return;
    const int d = (int)(i % a.vd);
    const int h = (int)((i / a.vd) % a.nH);
    const long long t = i / ((long long)a.vd * a.nH);
    float y;
    if (a.mix) {
        const int c = h / (a.nH / a.nKV);
        y = 0.f;
        for (int g = 0; g < a.nH; ++g)
            y = fmaf(a.mix[h * a.nH + g], a.pairs[(((size_t)t * a.nH + g) * a.nKV + c) * a.vd + d], y);
    } else {
        y = a.pairs[((size_t)t * a.nH + h) * a.vd + d];
    }
    gl_store((TA*)a.out + i, y);
}

template <typename TA, typename TC, int NACC>
static int launch_mixed(const MixedAttnArgs& a, cudaStream_t stream) {
    const int pairs = a.nH * (a.mix ? a.nKV : 1);
    int rc;
    // the kernel by key head: with a table every query head of the key head in one block (up to eight, and a warp a
    // value head); without one, runs of eight query heads whose value heads are whole within a run or span whole runs
    const int group = a.nH / a.nKV, share = a.nH / am_value_heads(a);
    const bool by_key_head = a.mix ? (group <= 8 && a.nKV <= AM_GTHREADS / 32)
                                   : (group <= 8 ? group % (share < group ? share : group) == 0
                                                 : (group % 8 == 0 && (share >= 8 ? share % 8 == 0 : 8 % share == 0)));
    if (a.max_qlen == 1 && by_key_head && NACC <= 4 && a.parts && a.ml && a.splits > 0) {
        rc = launch_group_decode<TA, TC, NACC>(a, stream);
        if (rc != 0) return rc;
        return gl_launch(head_mix_split_kernel<TA>, dim3(a.nH, a.B), dim3(a.vd <= 64 ? 64 : 128), (size_t)(a.mix ? a.nH : 1) * a.splits * sizeof(float), stream, 1, a);
    } else if (a.max_qlen == 1) {
        const size_t smem = ((size_t)a.hd + (size_t)AM_DWARPS * (a.vd + 2)) * sizeof(float);
        rc = gl_launch(attn_pairs_decode_kernel<TA, TC, NACC>, dim3(pairs, a.B), dim3(AM_DWARPS * 32), smem, stream, 1, a);
    } else {
        size_t smem = ((size_t)GL_PAGE * (a.hd + 1) + (size_t)GL_PAGE * a.vd + (size_t)AM_ROWS * a.hd) * sizeof(float);
        int stage_rows = GL_PAGE;
        if (smem > 200 * 1024) {                    // long key rows: half a page of them at a time
            stage_rows = 32;
            smem = ((size_t)32 * (a.hd + 1) + (size_t)32 * a.vd + (size_t)AM_ROWS * a.hd) * sizeof(float);
        }
        auto kern = attn_pairs_kernel<TA, TC, NACC>;
        if (smem > 48 * 1024) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
                cudaGetLastError();
                return GL_ERR_SMEM;
            }
        }
        rc = gl_launch(kern, dim3((a.max_qlen + AM_ROWS - 1) / AM_ROWS, pairs, a.B), dim3(AM_ROWS * 32), smem, stream, 1, a, stage_rows);
    }
    if (rc != 0) return rc;
    const long long n = (long long)a.T * a.nH * a.vd;
    return gl_launch(head_mix_kernel<TA>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, a);
}

// the kernel that puts a one-token step's ranges together, behind a kernel of another library that left them
GL_API int gl_head_mix_split(const MixedAttnArgs* args, int act_dtype, cudaStream_t stream) {
    const MixedAttnArgs& a = *args;
    if (a.B <= 0) return GL_OK;
    if (!a.parts || !a.ml || a.splits <= 0 || a.vd <= 0) return GL_ERR_SHAPE;
    const dim3 grid(a.nH, a.B), block(a.vd <= 64 ? 64 : 128);
    const size_t smem = (size_t)(a.mix ? a.nH : 1) * a.splits * sizeof(float);
    int rc;
    if (act_dtype == GL_F32) rc = gl_launch(head_mix_split_kernel<float>, grid, block, smem, stream, 1, a);
    else if (act_dtype == GL_BF16) rc = gl_launch(head_mix_split_kernel<__nv_bfloat16>, grid, block, smem, stream, 1, a);
    else return GL_ERR_DTYPE;
    return rc == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// the mixing kernel alone, behind a pairs kernel of another library
GL_API int gl_head_mix(const MixedAttnArgs* args, int act_dtype, cudaStream_t stream) {
    const MixedAttnArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    const long long n = (long long)a.T * a.nH * a.vd;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (act_dtype == GL_F32) return gl_launch(head_mix_kernel<float>, grid, dim3(256), 0, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
    if (act_dtype == GL_BF16) return gl_launch(head_mix_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
    return GL_ERR_DTYPE;
}

template <typename TA, typename TC>
static int dispatch_mixed(const MixedAttnArgs& a, cudaStream_t stream) {
    switch ((a.vd + 31) / 32) {
        case 1: return launch_mixed<TA, TC, 1>(a, stream);
        case 2: return launch_mixed<TA, TC, 2>(a, stream);
        case 3: return launch_mixed<TA, TC, 3>(a, stream);
        case 4: return launch_mixed<TA, TC, 4>(a, stream);
        case 5: return launch_mixed<TA, TC, 5>(a, stream);
        case 6: return launch_mixed<TA, TC, 6>(a, stream);
        case 7: return launch_mixed<TA, TC, 7>(a, stream);
        case 8: return launch_mixed<TA, TC, 8>(a, stream);
        default: return GL_ERR_SHAPE;
    }
}

GL_API int gl_attention_mixed(const MixedAttnArgs* args, int act_dtype, int cache_dtype, cudaStream_t stream) {
    const MixedAttnArgs& a = *args;
    if (a.B <= 0 || a.max_qlen <= 0 || a.T <= 0) return GL_OK;
    if (a.hd <= 0 || a.hd > 1024 || a.vd <= 0 || a.vd > 256 || a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV) return GL_ERR_SHAPE;
    if (a.nVH < 0 || (a.nVH > 0 && (a.nVH % a.nKV || a.nH % a.nVH || (a.mix && a.nVH != a.nKV)))) return GL_ERR_SHAPE;
    if (a.vs < 0 || (a.vs > 0 && a.vs < a.vd)) return GL_ERR_SHAPE;
    if (a.B > 65535 || a.nH * a.nKV > 65535) return GL_ERR_SHAPE;
    if (act_dtype == GL_F32 && cache_dtype == GL_F32) return dispatch_mixed<float, float>(a, stream);
    if (act_dtype == GL_BF16 && cache_dtype == GL_BF16) return dispatch_mixed<__nv_bfloat16, __nv_bfloat16>(a, stream);
    return GL_ERR_DTYPE;
}
