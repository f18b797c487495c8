// Prompt attention for a mixer whose heads' softmax weights are mixed before they meet the values
// (see attention_mixed.cu): the pairs A[g, c](i) = sum_j p_g(i, j) v_c(j) on the tensor cores, bfloat16.
//
// A block takes 64 consecutive query rows of one pair (query head g, value head c) of one sequence; each
// of its 4 warps owns 16 rows.  Key pages of g's key head and value pages of head c (64 positions each)
// stream through shared memory with cp.async, two pages in flight.  Scores and the output are
// mma.sync.m16n8k16 products with 32-bit accumulators; the maximum, the sum, the weights and the
// rescaling of the running softmax are 32-bit, and the pair's result leaves in 32-bit for the mixing
// kernel.  Rows past a sequence's length are zero-filled on load.  Key and value sizes are compile-time
// constants (GL_HEAD_DIM, GL_VALUE_DIM), multiples of 16.
#include "common.cuh"

#ifndef GL_HEAD_DIM
#error "compile with -DGL_HEAD_DIM=<key size> [-DGL_VALUE_DIM=<value size>]"
#endif
#ifndef GL_VALUE_DIM
#define GL_VALUE_DIM GL_HEAD_DIM
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 256, "key size: 16..256 in steps of 16");
static_assert(GL_VALUE_DIM % 16 == 0 && GL_VALUE_DIM >= 16 && GL_VALUE_DIM <= 256, "value size: 16..256 in steps of 16");

#define AP_HD GL_HEAD_DIM
#define AP_VD GL_VALUE_DIM
#define AP_BM 64
#define AP_THREADS 128
#define AP_KS (AP_HD / 16)            // k-steps of the score product
#define AP_NT (AP_VD / 8)             // 8-wide column tiles of the output
#define AP_ROW (AP_HD * 2 + 16)       // padded row: 8 consecutive rows fall in distinct banks
#define AP_VROW (AP_VD * 2 + 16)
#define AP_TILE (64 * AP_ROW)
#define AP_VTILE (64 * AP_VROW)

struct PairsArgs {
    const void* q;            // [T, nH*hd] bf16, already scaled
    float* pairs;             // [T, nH, nVal, vd] 32-bit
    const void* k_cache;      // [pages, nKV, GL_PAGE, hd] bf16
    const void* v_cache;      // [pages, nKV, GL_PAGE, vd] bf16
    const int* seq_qstart;    // [B]
    const int* seq_qlen;      // [B]
    const int* seq_ctx;       // [B]
    const int* pages;         // [B, max_pages]
    int B, nH, nKV, nVal, max_pages, window, max_qlen;
    float score_scale;        // multiplies q . k
    float softcap;            // > 0: s <- softcap * tanh(s / softcap)
    const float* slopes;      // [nH] or null: s <- s - slope_h * (query position - key position)
    void* out;                // [T, nH*vd] bf16 or null: without a mixing table (nVal 1) the result goes here, rounded,
                              // and no second kernel has to read the 32-bit pairs again
    const float* sinks;       // [nH] or null: e^(sinks[h]) joins the softmax's denominator of head h
    int nVH;                  // heads of the value cache where they are more than the key heads (0: nKV); without a
                              // table, query head h then takes the values of head h / (nH / nVH)
    int vs;                   // numbers between two positions' values of a head (0: the value size); a cache whose values
                              // are the first columns of its key rows is read with v_cache = k_cache and vs = the key size
    int v_in_k;               // such a cache with one row of values a key head: no value tile is fetched, the second
                              // product reads the key tile
};

__device__ __forceinline__ unsigned ap_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ap_cp16(unsigned dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ap_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void ap_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ap_ldm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_ldm4t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// cap * tanh(x / cap) as cap * (1 - 2 / (e^(2x/cap) + 1)) with the hardware's exponential and reciprocal: off by
// a few 1e-7 of cap (1e-5 at a cap of 50), which is small against what bfloat16 queries and keys leave in a score
// (2^-9 of it), and a fifth of the instructions of tanhf; every score of a prompt passes here, and with tanhf the
// shaping was most of what the kernel issued.  (The 32-bit kernels keep tanhf.)
__device__ __forceinline__ float ap_softcap(float x, float cap, float two_over_cap) {
    const float e = __expf(x * two_over_cap);                 // inf for large x: the quotient is then 0
    return cap * (1.0f - __fdividef(2.0f, e + 1.0f));
}
__device__ __forceinline__ unsigned ap_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// rows [0, n_valid) of a page tile (or of the query tile) to padded shared memory; the rest is zero
template <int DIM>
__device__ __forceinline__ void ap_load_rows(unsigned dst, const __nv_bfloat16* src, size_t src_row_stride, int n_valid) {
    constexpr int CHUNKS = DIM / 8, ROW = DIM * 2 + 16;
    for (int i = threadIdx.x; i < 64 * CHUNKS; i += AP_THREADS) {
        const int r = i / CHUNKS, c = i - r * CHUNKS;
        const bool ok = r < n_valid;
        ap_cp16(dst + r * ROW + c * 16, ok ? (const void*)(src + (size_t)r * src_row_stride + c * 8) : (const void*)src,
                ok ? 16 : 0);
    }
}

__global__ void __launch_bounds__(AP_THREADS)
attn_pairs_tc_kernel(PairsArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    // (the query tile passes through the second key stage before the first page is asked for: a block's shared
    // memory is two key stages and two value stages, so that two or three blocks fit an SM at long key rows)
    const unsigned sK[2] = {ap_smem(smem), ap_smem(smem) + AP_TILE};
    const unsigned sQ = sK[1];
    const unsigned sV[2] = {sK[0] + 2 * AP_TILE, sK[0] + 2 * AP_TILE + AP_VTILE};
    gl_grid_wait();                                            // (a long kernel: the next one is not launched early)
    const int b = blockIdx.z;
    const int h = blockIdx.y / a.nVal;                         // query head
    const int g = h / (a.nH / a.nKV);                          // its key head
    const int nvh = a.nVH > 0 ? a.nVH : a.nKV;
    const int vh = a.nVal > 1 ? blockIdx.y - h * a.nVal : h / (a.nH / nvh);   // the pair's value head
    const int qlen = a.seq_qlen[b];
    const int n_qtiles = (qlen + AP_BM - 1) / AP_BM;
    const int qt = n_qtiles - 1 - (int)blockIdx.x;           // longest rows first
    if (qt < 0) return;
    const int ctx = a.seq_ctx[b], qstart = a.seq_qstart[b];
    const int q0 = qt * AP_BM;
    const int rows = min(AP_BM, qlen - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane >> 2, t = lane & 3;
    const int p_first = ctx + q0, p_last = ctx + q0 + rows - 1;
    const int lo_first = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
    const int page_begin = lo_first / GL_PAGE, page_end = p_last / GL_PAGE + 1;
    const int* pg = a.pages + (size_t)b * a.max_pages;
    const __nv_bfloat16* K = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* V = (const __nv_bfloat16*)a.v_cache;
    const size_t head_off = (size_t)g * GL_PAGE * AP_HD, page_stride = (size_t)a.nKV * GL_PAGE * AP_HD;
    const size_t vs = a.vs > 0 ? (size_t)a.vs : (size_t)AP_VD;
    const size_t vhead_off = (size_t)vh * GL_PAGE * vs, vpage_stride = (size_t)nvh * GL_PAGE * vs;
    const int total = ctx + qlen;

    // the query tile and the first page; the tile's fragments go to registers before its stage is used for keys
    ap_load_rows<AP_HD>(sQ, (const __nv_bfloat16*)a.q + ((size_t)(qstart + q0) * a.nH + h) * AP_HD, (size_t)a.nH * AP_HD, rows);
    {
        const int nv = min(GL_PAGE, total - page_begin * GL_PAGE);
        ap_load_rows<AP_HD>(sK[0], K + (size_t)pg[page_begin] * page_stride + head_off, AP_HD, nv);
        if (!a.v_in_k) ap_load_rows<AP_VD>(sV[0], V + (size_t)pg[page_begin] * vpage_stride + vhead_off, vs, nv);
    }
    ap_commit();
    ap_wait<0>();
    __syncthreads();

    unsigned qf[AP_KS][4];
#pragma unroll
    for (int kk = 0; kk < AP_KS; ++kk) {
        const int r = (threadIdx.x >> 5) * 16 + (threadIdx.x & 7) + ((threadIdx.x >> 3) & 1) * 8;
        const int c = kk * 2 + ((threadIdx.x & 31) >> 4);
        ap_ldm4(sQ + r * AP_ROW + c * 16, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
    __syncthreads();
    float o[AP_NT][4];
#pragma unroll
    for (int i = 0; i < AP_NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;
    const float slope = a.slopes ? a.slopes[h] : 0.f;
    const bool shaped = a.score_scale != 1.0f || a.softcap > 0.f || a.slopes != nullptr;
    const float two_over_cap = a.softcap > 0.f ? 2.0f / a.softcap : 0.f;
    const int r_lo = warp * 16 + grp, r_hi = r_lo + 8;        // this thread's two rows inside the tile
    const int pos_lo = p_first + r_lo, pos_hi = p_first + r_hi;
    const int wlo_lo = (a.window > 0 && pos_lo - a.window + 1 > 0) ? pos_lo - a.window + 1 : 0;
    const int wlo_hi = (a.window > 0 && pos_hi - a.window + 1 > 0) ? pos_hi - a.window + 1 : 0;

    for (int p = page_begin; p < page_end; ++p) {
        const int st = (p - page_begin) & 1;
        if (p + 1 < page_end) {
            const int nv = min(GL_PAGE, total - (p + 1) * GL_PAGE);
            ap_load_rows<AP_HD>(sK[st ^ 1], K + (size_t)pg[p + 1] * page_stride + head_off, AP_HD, nv);
            if (!a.v_in_k) ap_load_rows<AP_VD>(sV[st ^ 1], V + (size_t)pg[p + 1] * vpage_stride + vhead_off, vs, nv);
        }
        ap_commit();
        ap_wait<1>();
        __syncthreads();
        const int j0 = p * GL_PAGE;
        // a warp whose rows all lie before this page has nothing to do here (causal)
        const bool warp_active = j0 <= p_first + warp * 16 + 15;
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < AP_KS; ++kk) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    unsigned b0, b1, b2, b3;
                    const int r = j * 8 + ((lane >> 4) & 1) * 8 + (lane & 7);
                    const int c = kk * 2 + ((lane >> 3) & 1);
                    ap_ldm4(sK[st] + r * AP_ROW + c * 16, b0, b1, b2, b3);
                    ap_mma(s[j], qf[kk], b0, b1);
                    ap_mma(s[j + 1], qf[kk], b2, b3);
                }
            }
            if (shaped) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = j0 + j * 8 + 2 * t + (e & 1);
                        float x = s[j][e] * a.score_scale;
                        if (a.softcap > 0.f) x = ap_softcap(x, a.softcap, two_over_cap);
                        s[j][e] = x - slope * (float)(((e < 2) ? pos_lo : pos_hi) - key);
                    }
                }
            }
            // mask: a row at position x sees keys max(0, x-window+1) .. x
            const bool need_mask = (j0 + GL_PAGE - 1 > p_first + warp * 16) || (a.window > 0 && j0 < wlo_hi + 8);
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = j0 + j * 8 + 2 * t + (e & 1);
                        const int pos = (e < 2) ? pos_lo : pos_hi;
                        const int wl = (e < 2) ? wlo_lo : wlo_hi;
                        if (key > pos || key < wl) s[j][e] = -INFINITY;
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            }
            float corr[2], mu[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_new = fmaxf(m_run[i], mx[i]);
                mu[i] = (m_new == -INFINITY) ? 0.f : m_new * LOG2E;
                corr[i] = exp2f(m_run[i] * LOG2E - mu[i]);       // m_run = -inf gives 0
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][0] = exp2f(s[j][0] * LOG2E - mu[0]);
                s[j][1] = exp2f(s[j][1] * LOG2E - mu[0]);
                s[j][2] = exp2f(s[j][2] * LOG2E - mu[1]);
                s[j][3] = exp2f(s[j][3] * LOG2E - mu[1]);
                l_run[0] += s[j][0] + s[j][1];
                l_run[1] += s[j][2] + s[j][3];
            }
#pragma unroll
            for (int i = 0; i < AP_NT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                unsigned pa[4];
                pa[0] = ap_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = ap_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = ap_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = ap_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dn = 0; dn < AP_NT; dn += 2) {
                    unsigned b0, b1, b2, b3;
                    const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int c = dn + (lane >> 4);
                    ap_ldm4t((a.v_in_k ? sK[st] + r * AP_ROW : sV[st] + r * AP_VROW) + c * 16, b0, b1, b2, b3);
                    ap_mma(o[dn], pa, b0, b1);
                    ap_mma(o[dn + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    ap_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    float inv_lo = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
    float inv_hi = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    if (a.sinks) {
        // the sink joins the denominator once, against the larger of the row's maximum and itself
        const float sink = a.sinks[h];
        const float top_lo = fmaxf(m_run[0], sink), top_hi = fmaxf(m_run[1], sink);
        const float sc_lo = m_run[0] > -INFINITY ? expf(m_run[0] - top_lo) : 0.f;
        const float sc_hi = m_run[1] > -INFINITY ? expf(m_run[1] - top_hi) : 0.f;
        inv_lo = sc_lo / (l_run[0] * sc_lo + expf(sink - top_lo));
        inv_hi = sc_hi / (l_run[1] * sc_hi + expf(sink - top_hi));
    }
    const int slot = a.nVal > 1 ? vh : 0;
    if (a.out && a.nVal == 1) {
        __nv_bfloat16* O = (__nv_bfloat16*)a.out;
#pragma unroll
        for (int i = 0; i < AP_NT; ++i) {
            const int d = i * 8 + 2 * t;
            if (r_lo < rows)
                *(__nv_bfloat162*)(O + ((size_t)(qstart + q0 + r_lo) * a.nH + h) * AP_VD + d) =
                    __floats2bfloat162_rn(o[i][0] * inv_lo, o[i][1] * inv_lo);
            if (r_hi < rows)
                *(__nv_bfloat162*)(O + ((size_t)(qstart + q0 + r_hi) * a.nH + h) * AP_VD + d) =
                    __floats2bfloat162_rn(o[i][2] * inv_hi, o[i][3] * inv_hi);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < AP_NT; ++i) {
        const int d = i * 8 + 2 * t;
        if (r_lo < rows)
            *(float2*)(a.pairs + (((size_t)(qstart + q0 + r_lo) * a.nH + h) * a.nVal + slot) * AP_VD + d) =
                make_float2(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (r_hi < rows)
            *(float2*)(a.pairs + (((size_t)(qstart + q0 + r_hi) * a.nH + h) * a.nVal + slot) * AP_VD + d) =
                make_float2(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

// ---------------------------------------------------------------------------
// One token a sequence, many query heads on one key head (every head of a mixer that reads one wide key row per
// position): the heads are the rows of the score product.  A block takes a run of up to 16 query heads that share a
// value head, one sequence and a range of its pages; K and V pages stream through shared memory with cp.async, two
// in flight; warp w owns keys 16w..16w+15 of every page with a running softmax of its own, S = Q K^T and O += P V on
// mma.sync.m16n8k16, 32-bit softmax; the four warps' results are put together in shared memory and leave as the
// range's sums not yet divided, with its maximum and sum, for the kernel that merges the ranges
// (head_mix_split_kernel in attention_mixed.cu, which also knows the sinks).  With v_in_k the values are the first
// AP_VD columns of the key rows and no value page is fetched at all.
// ---------------------------------------------------------------------------
struct RowsDecodeArgs {
    const void* q;            // [B rows, nH*hd] bf16
    const void* k_cache;      // [pages, nKV, GL_PAGE, hd] bf16
    const void* v_cache;      // [pages, nVH, GL_PAGE, vd] bf16 (unused with v_in_k)
    const int* seq_qstart;
    const int* seq_ctx;
    const int* pages;         // [B, max_pages]
    float* parts;             // [B, nH, 1, splits, vd] sums not yet divided
    float* ml;                // [B, nH, splits, 2] each range's maximum and sum
    int B, nH, nKV, nVH, max_pages, window, splits, pages_per_split, rows, v_in_k;
    float score_scale;
};

__global__ void __launch_bounds__(AP_THREADS)
attn_rows_decode_tc_kernel(RowsDecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int QT = 16 * AP_ROW;
    const unsigned sQ = ap_smem(smem);
    const unsigned sK[2] = {sQ + QT, sQ + QT + AP_TILE};
    const unsigned sV[2] = {sQ + QT + 2 * AP_TILE, sQ + QT + 2 * AP_TILE + AP_VTILE};
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.y, split = blockIdx.z;
    const int head0 = blockIdx.x * a.rows;
    const int kh = head0 / (a.nH / a.nKV), vh = head0 / (a.nH / a.nVH);
    const int p = a.seq_ctx[b];                                   // the token's position; keys lo..p
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int page_first = lo / GL_PAGE + split * a.pages_per_split;
    const int page_last = min(p / GL_PAGE, page_first + a.pages_per_split - 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane >> 2, t = lane & 3;
    const int* pg = a.pages + (size_t)b * a.max_pages;
    const __nv_bfloat16* K = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* V = (const __nv_bfloat16*)a.v_cache;
    const size_t head_off = (size_t)kh * GL_PAGE * AP_HD, page_stride = (size_t)a.nKV * GL_PAGE * AP_HD;
    const size_t vhead_off = (size_t)vh * GL_PAGE * AP_VD, vpage_stride = (size_t)a.nVH * GL_PAGE * AP_VD;

    // the run's queries: rows of heads; rows past the run are zero
    {
        const __nv_bfloat16* src = (const __nv_bfloat16*)a.q + ((size_t)a.seq_qstart[b] * a.nH + head0) * AP_HD;
        constexpr int CHUNKS = AP_HD / 8;
        for (int i = threadIdx.x; i < 16 * CHUNKS; i += AP_THREADS) {
            const int r = i / CHUNKS, c = i - r * CHUNKS;
            const bool ok = r < a.rows;
            ap_cp16(sQ + r * AP_ROW + c * 16, ok ? (const void*)(src + (size_t)r * AP_HD + c * 8) : (const void*)src, ok ? 16 : 0);
        }
    }
    auto fetch = [&](int page_i, int st) {
        const int nv = min(GL_PAGE, p + 1 - page_i * GL_PAGE);    // keys past p were never written
        ap_load_rows<AP_HD>(sK[st], K + (size_t)pg[page_i] * page_stride + head_off, AP_HD, nv);
        if (!a.v_in_k) ap_load_rows<AP_VD>(sV[st], V + (size_t)pg[page_i] * vpage_stride + vhead_off, AP_VD, nv);
    };
    if (page_first <= page_last) fetch(page_first, 0);
    ap_commit();

    float o[AP_NT][4];
#pragma unroll
    for (int i = 0; i < AP_NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;

    for (int pi = page_first; pi <= page_last; ++pi) {
        const int st = (pi - page_first) & 1;
        if (pi + 1 <= page_last) fetch(pi + 1, st ^ 1);
        ap_commit();
        ap_wait<1>();
        __syncthreads();
        const int j0 = pi * GL_PAGE + warp * 16;                   // this warp's first key of the page
        if (j0 <= p && j0 + 15 >= lo) {
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < AP_KS; ++kk) {
                unsigned qf[4], b0, b1, b2, b3;
                {
                    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int c = kk * 2 + (lane >> 4);
                    ap_ldm4(sQ + r * AP_ROW + c * 16, qf[0], qf[1], qf[2], qf[3]);
                }
                const int r = warp * 16 + ((lane >> 4) & 1) * 8 + (lane & 7);
                const int c = kk * 2 + ((lane >> 3) & 1);
                ap_ldm4(sK[st] + r * AP_ROW + c * 16, b0, b1, b2, b3);
                ap_mma(s[0], qf, b0, b1);
                ap_mma(s[1], qf, b2, b3);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j0 + j * 8 + 2 * t + (e & 1);
                    const float x = (key >= lo && key <= p) ? s[j][e] * a.score_scale : -INFINITY;
                    s[j][e] = x;
                    mx[e >> 1] = fmaxf(mx[e >> 1], x);
                }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            }
            float corr[2], mu[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_new = fmaxf(m_run[i], mx[i]);
                mu[i] = (m_new == -INFINITY) ? 0.f : m_new * LOG2E;
                corr[i] = exp2f(m_run[i] * LOG2E - mu[i]);          // m_run = -inf gives 0
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][0] = exp2f(s[j][0] * LOG2E - mu[0]);
                s[j][1] = exp2f(s[j][1] * LOG2E - mu[0]);
                s[j][2] = exp2f(s[j][2] * LOG2E - mu[1]);
                s[j][3] = exp2f(s[j][3] * LOG2E - mu[1]);
                l_run[0] += s[j][0] + s[j][1];
                l_run[1] += s[j][2] + s[j][3];
            }
#pragma unroll
            for (int i = 0; i < AP_NT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
            unsigned pa[4];
            pa[0] = ap_pack(s[0][0], s[0][1]);
            pa[1] = ap_pack(s[0][2], s[0][3]);
            pa[2] = ap_pack(s[1][0], s[1][1]);
            pa[3] = ap_pack(s[1][2], s[1][3]);
            const unsigned vbase = a.v_in_k ? sK[st] : sV[st];
            const int vrow = a.v_in_k ? AP_ROW : AP_VROW;
#pragma unroll
            for (int dn = 0; dn < AP_NT; dn += 2) {
                unsigned b0, b1, b2, b3;
                const int r = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int c = dn + (lane >> 4);
                ap_ldm4t(vbase + r * vrow + c * 16, b0, b1, b2, b3);
                ap_mma(o[dn], pa, b0, b1);
                ap_mma(o[dn + 1], pa, b2, b3);
            }
        }
        __syncthreads();
    }
    ap_wait<0>();
    __syncthreads();
    // the four warps' sums, maxima and sums of weights side by side in shared memory (over the page stages)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    float* po = (float*)(smem + QT);                              // [4][16][AP_VD]
    float* pm = po + 4 * 16 * AP_VD;                              // [4][16][2]
#pragma unroll
    for (int i = 0; i < AP_NT; ++i) {
        const int d = i * 8 + 2 * t;
        *(float2*)(po + ((size_t)warp * 16 + grp) * AP_VD + d) = make_float2(o[i][0], o[i][1]);
        *(float2*)(po + ((size_t)warp * 16 + grp + 8) * AP_VD + d) = make_float2(o[i][2], o[i][3]);
    }
    if (t == 0) {
        pm[(warp * 16 + grp) * 2] = m_run[0];
        pm[(warp * 16 + grp) * 2 + 1] = l_run[0];
        pm[(warp * 16 + grp + 8) * 2] = m_run[1];
        pm[(warp * 16 + grp + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.rows * AP_VD; i += AP_THREADS) {
        const int r = i / AP_VD, d = i - r * AP_VD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, pm[(w * 16 + r) * 2]);
        float y = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = pm[(w * 16 + r) * 2];
            if (mw > -INFINITY) {
                const float f = expf(mw - mm);
                y = fmaf(po[((size_t)w * 16 + r) * AP_VD + d], f, y);
                l = fmaf(pm[(w * 16 + r) * 2 + 1], f, l);
            }
        }
        a.parts[(((size_t)b * a.nH + head0 + r) * a.splits + split) * AP_VD + d] = y;
        if (d == 0) {
            float* dst = a.ml + (((size_t)b * a.nH + head0 + r) * a.splits + split) * 2;
            dst[0] = mm;
            dst[1] = l;
        }
    }
}

GL_API int gl_attention_rows_decode_tc(const RowsDecodeArgs* args, cudaStream_t stream) {
    const RowsDecodeArgs& a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.nH <= 0 || a.nKV <= 0 || a.nVH <= 0 || a.nH % a.nKV || a.nH % a.nVH || a.rows <= 0 || a.rows > 16 || a.nH % a.rows ||
        (a.nH / a.nVH) % a.rows || (a.nH / a.nKV) % a.rows || a.splits <= 0 || a.pages_per_split <= 0) return GL_ERR_SHAPE;
    if (a.v_in_k && (AP_VD > AP_HD || a.nVH != a.nKV)) return GL_ERR_SHAPE;
    if (a.B > 65535 || a.splits > 65535) return GL_ERR_SHAPE;
    const size_t stages = 16 * (size_t)AP_ROW + 2 * (size_t)AP_TILE + (a.v_in_k ? 0 : 2 * (size_t)AP_VTILE);
    const size_t merge = 16 * (size_t)AP_ROW + (4 * 16 * (size_t)AP_VD + 4 * 16 * 2) * sizeof(float);
    const size_t smem = stages > merge ? stages : merge;
    if (smem > 227 * 1024) return GL_ERR_SMEM;
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(attn_rows_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = smem;
    }
    dim3 grid(a.nH / a.rows, a.B, a.splits);
    return gl_launch(attn_rows_decode_tc_kernel, grid, dim3(AP_THREADS), smem, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

GL_API int gl_attention_pairs_tc_dims() { return AP_HD * 1000 + AP_VD; }

GL_API int gl_attention_pairs_tc(const PairsArgs* args, cudaStream_t stream) {
    const PairsArgs& a = *args;
    if (a.B <= 0 || a.max_qlen <= 0) return GL_OK;
    if (a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV || (a.nVal != 1 && a.nVal != a.nKV)) return GL_ERR_SHAPE;
    if (a.nVH < 0 || (a.nVH > 0 && (a.nH % a.nVH || (a.nVal != 1 && a.nVH != a.nKV)))) return GL_ERR_SHAPE;
    if (a.vs < 0 || (a.vs > 0 && (a.vs < AP_VD || a.vs % 8))) return GL_ERR_SHAPE;
    if (a.v_in_k && (AP_VD > AP_HD || a.nVal != 1 || (a.nVH > 0 && a.nVH != a.nKV))) return GL_ERR_SHAPE;
    if (a.B > 65535 || a.nH * a.nVal > 65535) return GL_ERR_SHAPE;
    const size_t smem = 2 * (size_t)AP_TILE + (a.v_in_k ? 0 : 2 * (size_t)AP_VTILE);
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(attn_pairs_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = smem;
    }
    dim3 grid((a.max_qlen + AP_BM - 1) / AP_BM, a.nH * a.nVal, a.B);
    return gl_launch(attn_pairs_tc_kernel, grid, dim3(AP_THREADS), smem, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}
