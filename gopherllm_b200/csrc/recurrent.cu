// Mixers that carry a fixed-size state from token to token instead of a growing cache:
// matrix memories with outer-product updates (an exponentially gated one with a normaliser and a
// running maximum, and one whose per-channel forget gate also sets what is written) and a
// selective state-space scan behind a short causal convolution.
//
// A step brings, for every sequence of the batch, a run of one or more tokens; the state of a
// sequence lives in its row of a 32-bit table (row = the sequence's slot), is read when the run
// starts and written back when it ends, so a prompt gives the same result whole, in pieces or token
// by token.  Everything that enters a recurrence (gates, decays, step sizes, the state itself) is
// 32-bit; the projections that feed it arrive in the activation type.
//
// The scans walk a run's tokens in order.  Work is spread over what is independent: sequences,
// heads and the columns of a memory (or the channels of the scan); a thread keeps its part of the
// state in registers for the whole run, and the tokens' inputs are staged in shared memory a few
// tokens at a time.
#include "common.cuh"

#define RC_THREADS 128
#define MS_THREADS 256     // the matrix memories' blocks
#define SS_CHUNK 16         // tokens the selective scan stages at a time

__device__ __forceinline__ float rc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float rc_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float rc_log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float rc_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
// e^x for a decay that is applied at every token: near one the factor comes from expm1f, which is
// rounded once; expf's last-bit errors near one do not average out over a thousand tokens of a slowly
// decaying state.
__device__ __forceinline__ float rc_decay(float x) {
    if (x > -0.5f && x <= 0.f) {
        // 1 + (e^x - 1) with e^x - 1 from its series to x^9/9! (below 2^-28 here), Horner in 32-bit
        float p = 2.755731922e-6f;
        p = fmaf(p, x, 2.48015873e-5f);
        p = fmaf(p, x, 1.984126984e-4f);
        p = fmaf(p, x, 1.388888889e-3f);
        p = fmaf(p, x, 8.333333333e-3f);
        p = fmaf(p, x, 4.166666667e-2f);
        p = fmaf(p, x, 1.666666667e-1f);
        p = fmaf(p, x, 0.5f);
        p = fmaf(p, x, 1.0f);
        return fmaf(p, x, 1.0f);
    }
    if (x > -0.5f) return 1.0f + expm1f(x);
    return expf(x);
}

// ---------------------------------------------------------------------------
// Matrix memories.  Per head a state S [D, V]; a token's output is S^T q.
//   kind 0, gated with a normaliser: log gates gi = cap tanh(i/cap), gf = logsigmoid(cap tanh(f/cap));
//       m' = max(gf + m, gi);  S' = e^(gf+m-m') S + e^(gi-m') k v^T;  n' likewise with k alone;
//       o = S'^T q / (max(|n'.q|, e^(-m')) + 1e-6).     m starts at 0 (a zeroed state row).
//   kind 1, forget gate with a lower bound: f = l + (1-l) sigmoid(fpre) per row;
//       S' = diag(f) S + (1-f) v^T;  o = S'^T q,  q = silu(qpre).
//   kind 2, gated delta rule: q and k (shared by H / KVH heads) brought to unit length, x / sqrt(sum x^2 + 1e-6),
//       q times q_scale; beta = sigmoid(b), g = e^(-e^(A_log) softplus(a + dt_bias)) per head, from a second
//       tensor of projections (``gates``: b at column i_off + h, a at f_off + h);
//       S <- g S;  u = beta (v - S^T k);  S' = S + k u^T;  o = S'^T q.
//   kind 3, plain decay: S' = keep S + take k v^T;  o = S'^T q + skip_h v.  q and k (shared by H / KVH heads) may be
//       rotated by the token's position first (the first 2 rot_half dims of a head, dim i paired with i + rot_half,
//       cosines and sines [T, rot_half] of the step's tokens) and are then scaled by q_scale and k_scale.  The
//       decay is fixed per head (keep = lower[h], take = 1: retention) or follows a step size from a second tensor
//       of projections (``gates``, column f_off + h): dt = softplus(x + dt_bias[h]), keep = e^(-e^(A_log[h]) dt),
//       take = dt (a state-space layer with a scalar decay per head, whose B, x, C are this memory's k, v, q).
// State row: S [H, D, V], then for kind 0 n [H, D] and m [H].  Every block of a head's columns reads n and m
// when it starts, and blocks of one head may run one after the other, so the new n and m go to a scratch
// [B, H, D + 1] first and a second kernel moves them into the rows once all blocks are done.
// ---------------------------------------------------------------------------
struct MemoryScanArgs {
    const void* proj;         // [T, ld] activation type: the joined projections of the step's tokens
    float* out;               // [T, H*V] 32-bit
    float* state;             // [slots, state_stride]
    const float* lower;       // kind 1: [H*D] lower bounds of the forget gate
    const int* seq_slot;      // [B]
    const int* seq_qstart;    // [B]
    const int* seq_qlen;      // [B]
    int ld, q_off, k_off, v_off, i_off, f_off;
    int B, H, D, V, state_stride, kind;
    float cap, q_scale;
    float* nm_next;           // kind 0: [B, H, D + 1] scratch for the new normaliser and maximum
    // kind 2:
    const void* gates;        // [T, gates_ld] activation type: the projections behind beta and the decay
    const float* a_log;       // [H]
    const float* dt_bias;     // [H]
    int gates_ld, KVH;        // KVH: heads of q and k (each shared by H / KVH heads of v)
    int rows_per_thread;      // 0: chosen by the grid's size; else 32, 8, 4, 2 or 1 (for measurements)
    // kind 3:
    const float* cosv;        // [T, rot_half] or null: q and k are rotated by the token's position
    const float* sinv;
    int rot_half;
    float k_scale;            // multiplies k after the rotation
    const float* d_skip;      // [H] or null: o += d_skip[h] * v
};

// FULL: D == R * DPT and D a multiple of 4, so a thread's rows are DPT / 4 groups of four consecutive ones read
// as float4 and no row needs a bounds check.
template <typename TA, int DPT, int KIND, bool FULL>
__global__ void __launch_bounds__(MS_THREADS)
memory_scan_kernel(MemoryScanArgs a, int R, int CH) {
    extern __shared__ __align__(16) float smem[];
    // (launched in order, not early: placed beside the kernel before, the blocks of a scan sat several to an SM
    // for its whole length, and a prompt of 2,048 tokens took 25 ms instead of 16)
    gl_grid_wait();
    const int D = a.D, V = a.V, H = a.H;
    const int CT = MS_THREADS / R;                    // columns of a block
    const int b = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * CT;
    const int r = threadIdx.x % R, c = threadIdx.x / R;
    const int col = col0 + c;
    const bool live = col < V;
    const int qlen = a.seq_qlen[b], qstart = a.seq_qstart[b];
    float* qs = smem;                                 // [CHUNK][D]
    float* ks = qs + CH * D;                    // [CHUNK][D]   kind 0: k;  kind 1: f
    float* vs = ks + CH * D;                    // [CHUNK][CT]
    float* gs = vs + CH * CT;                   // [CHUNK][4]   kind 0: gi, gf, then keep, take; [.][3] reused
    float* es = gs + CH * 4;                    // [CHUNK]      kind 0: e^(-m')

    const int kh = (KIND == 2 || KIND == 3) ? h / (H / a.KVH) : h;   // the head of q and k this head reads
    float* srow = a.state + (size_t)a.seq_slot[b] * a.state_stride;
    float* S_g = srow + (size_t)h * D * V;
    const float* n_g = srow + (size_t)H * D * V + (size_t)h * D;
    const float* m_g = srow + (size_t)H * D * V + (size_t)H * D + h;
    float S[DPT], n[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = FULL ? ((((i >> 2) * R + r) << 2) + (i & 3)) : r + R * i;
        S[i] = (live && d < D) ? S_g[(size_t)d * V + col] : 0.f;
        n[i] = (KIND == 0 && d < D) ? n_g[d] : 0.f;
    }
    float m = KIND == 0 ? *m_g : 0.f;                 // only thread 0 keeps it current
    float* out_col = a.out + (size_t)qstart * H * V + (size_t)h * V + (live ? col : 0);
    float pending = 0.f;                              // kind 2: a token's read-out before its lanes are summed

    // The delta rule's inputs in bfloat16, rows of whole 16-byte units: a chunk's q, k, v and gate inputs are
    // asked for as 16-byte pieces while the chunk before is still being walked (they wait in registers), so that
    // a chunk's trip to memory does not stand between two walks.  (Fetched two bytes at a time behind the walk,
    // the staging of 32 tokens took longer than walking them.)
    constexpr int PIECES = 3;                         // CH * D <= 5120: at most 640 pieces of 8 for 256 threads
    const bool fast = KIND == 2 && sizeof(TA) == 2 && (a.ld % 8 == 0) && (a.q_off % 8 == 0) && (a.k_off % 8 == 0) &&
                      (a.v_off % 8 == 0) && (D % 8 == 0) && (V % 8 == 0) && (((uintptr_t)a.proj & 15) == 0) &&
                      CH * D <= PIECES * 8 * MS_THREADS;
    uint4 rq[PIECES], rk[PIECES], rv = make_uint4(0, 0, 0, 0);
    float rb = 0.f, ra = 0.f;
    auto fetch = [&](int s0) {
        const int ns = min(CH, qlen - s0), d8n = D / 8;
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int e = threadIdx.x + i * MS_THREADS;
            if (e < ns * d8n) {
                const int s = e / d8n, d8 = (e - s * d8n) * 8;
                const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
                rq[i] = *(const uint4*)(row + a.q_off + kh * D + d8);
                rk[i] = *(const uint4*)(row + a.k_off + kh * D + d8);
            }
        }
        const int c8n = CT / 8;
        if ((int)threadIdx.x < ns * c8n) {
            const int s = threadIdx.x / c8n, j8 = (threadIdx.x - s * c8n) * 8;
            const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
            rv = col0 + j8 < V ? *(const uint4*)(row + a.v_off + h * V + col0 + j8) : make_uint4(0, 0, 0, 0);
        }
        if ((int)threadIdx.x < ns) {
            const TA* row = (const TA*)a.gates + (size_t)(qstart + s0 + threadIdx.x) * a.gates_ld;
            rb = gl_load(row + a.i_off + h);
            ra = gl_load(row + a.f_off + h);
        }
    };
    auto spread = [](const uint4& r, float* dst) {
        const __nv_bfloat162* p2 = (const __nv_bfloat162*)&r;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p2[i]);
            dst[2 * i] = f.x;
            dst[2 * i + 1] = f.y;
        }
    };
    auto stash = [&](int ns) {
        const int d8n = D / 8, c8n = CT / 8;
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int e = threadIdx.x + i * MS_THREADS;
            if (e < ns * d8n) {
                spread(rq[i], qs + e * 8);
                spread(rk[i], ks + e * 8);
            }
        }
        if ((int)threadIdx.x < ns * c8n) spread(rv, vs + threadIdx.x * 8);
        if ((int)threadIdx.x < ns) {
            gs[threadIdx.x * 4 + 0] = rc_sigmoid(rb);
            gs[threadIdx.x * 4 + 1] = rc_decay(-expf(a.a_log[h]) * rc_softplus(ra + a.dt_bias[h]));
        }
    };
    if (fast && qlen > 0) fetch(0);

    for (int s0 = 0; s0 < qlen; s0 += CH) {
        const int ns = min(CH, qlen - s0);
        __syncthreads();
        if (fast) stash(ns);
#pragma unroll 4
        for (int e = threadIdx.x; !fast && e < ns * D; e += MS_THREADS) {
            const int s = e / D, d = e - s * D;
            const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
            const float qp = gl_load(row + a.q_off + kh * D + d);
            if (KIND == 0) {
                qs[e] = qp * a.q_scale;
                ks[e] = gl_load(row + a.k_off + h * D + d);
            } else if (KIND == 2) {
                qs[e] = qp;
                ks[e] = gl_load(row + a.k_off + kh * D + d);
            } else if (KIND == 3) {
                float qv = qp, kv = gl_load(row + a.k_off + kh * D + d);
                if (a.cosv && d < 2 * a.rot_half) {
                    // the pair (u, v) = (dim i, dim i + rot_half) becomes (u c - v s, v c + u s)
                    const bool first = d < a.rot_half;
                    const int i = first ? d : d - a.rot_half, other = first ? d + a.rot_half : d - a.rot_half;
                    const float c = a.cosv[(size_t)(qstart + s0 + s) * a.rot_half + i];
                    const float sn = a.sinv[(size_t)(qstart + s0 + s) * a.rot_half + i];
                    const float qo = gl_load(row + a.q_off + kh * D + other), ko = gl_load(row + a.k_off + kh * D + other);
                    qv = first ? qv * c - qo * sn : qv * c + qo * sn;
                    kv = first ? kv * c - ko * sn : kv * c + ko * sn;
                }
                qs[e] = qv * a.q_scale;
                ks[e] = kv * a.k_scale;
            } else {
                qs[e] = rc_silu(qp);
                const float l = a.lower[h * D + d];
                ks[e] = l + (1.0f - l) * rc_sigmoid(gl_load(row + a.f_off + h * D + d));
            }
        }
        for (int e = threadIdx.x; !fast && e < ns * CT; e += MS_THREADS) {
            const int s = e / CT, j = e - s * CT;
            const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
            vs[e] = col0 + j < V ? gl_load(row + a.v_off + h * V + col0 + j) : 0.f;
        }
        if (KIND == 2) {
            if (!fast && threadIdx.x < ns) {
                const TA* row = (const TA*)a.gates + (size_t)(qstart + s0 + threadIdx.x) * a.gates_ld;
                gs[threadIdx.x * 4 + 0] = rc_sigmoid(gl_load(row + a.i_off + h));
                gs[threadIdx.x * 4 + 1] = rc_decay(-expf(a.a_log[h]) * rc_softplus(gl_load(row + a.f_off + h) + a.dt_bias[h]));
            }
            __syncthreads();
            // unit length: a warp a token
            for (int s = threadIdx.x >> 5; s < ns; s += MS_THREADS / 32) {
                float sq = 0.f, sk = 0.f;
                for (int d = threadIdx.x & 31; d < D; d += 32) {
                    sq = fmaf(qs[s * D + d], qs[s * D + d], sq);
                    sk = fmaf(ks[s * D + d], ks[s * D + d], sk);
                }
                const float fq = a.q_scale / sqrtf(gl_warp_sum(sq) + 1e-6f), fk = 1.0f / sqrtf(gl_warp_sum(sk) + 1e-6f);
                for (int d = threadIdx.x & 31; d < D; d += 32) {
                    qs[s * D + d] *= fq;
                    ks[s * D + d] *= fk;
                }
            }
            if (fast && s0 + CH < qlen) fetch(s0 + CH);       // the next chunk's inputs travel while this one is walked
        }
        if (KIND == 3 && threadIdx.x < ns) {
            float take = 1.0f, keep = a.lower ? a.lower[h] : 1.0f;
            if (a.gates) {
                const TA* row = (const TA*)a.gates + (size_t)(qstart + s0 + threadIdx.x) * a.gates_ld;
                take = rc_softplus(gl_load(row + a.f_off + h) + a.dt_bias[h]);
                keep = rc_decay(-expf(a.a_log[h]) * take);
            }
            gs[threadIdx.x * 4 + 0] = take;
            gs[threadIdx.x * 4 + 1] = keep;
        }
        if (KIND == 0) {
            if (threadIdx.x < ns) {
                const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + threadIdx.x) * a.ld;
                gs[threadIdx.x * 4 + 0] = a.cap * tanhf(gl_load(row + a.i_off + h) / a.cap);
                gs[threadIdx.x * 4 + 1] = rc_log_sigmoid(a.cap * tanhf(gl_load(row + a.f_off + h) / a.cap));
            }
            __syncthreads();
            // the maximum is the only thing that goes from token to token here: one thread walks it, and the
            // tokens' factors are then taken side by side
            if (threadIdx.x == 0) {
                for (int s = 0; s < ns; ++s) {
                    const float m_new = fmaxf(gs[s * 4 + 1] + m, gs[s * 4 + 0]);
                    gs[s * 4 + 2] = m;
                    gs[s * 4 + 3] = m_new;
                    m = m_new;
                }
            }
            __syncthreads();
            if (threadIdx.x < ns) {
                const int s = threadIdx.x;
                const float gi = gs[s * 4 + 0], gf = gs[s * 4 + 1], m_old = gs[s * 4 + 2], m_new = gs[s * 4 + 3];
                gs[s * 4 + 2] = rc_decay(gf + m_old - m_new);
                gs[s * 4 + 3] = expf(gi - m_new);
                es[s] = expf(-m_new);
            }
        }
        __syncthreads();
#pragma unroll 4
        for (int s = 0; s < ns; ++s) {
            const float* q = qs + s * D;
            const float* k = ks + s * D;
            const float v = vs[s * CT + c];
            float num = 0.f, nq = 0.f;
            float qr[DPT], kr[DPT];
            if constexpr (FULL && DPT >= 4) {
#pragma unroll
                for (int i = 0; i < DPT; i += 4) {
                    // (a thread's rows are groups of four, R groups apart: the lanes of a column read consecutive
                    // 16-byte pieces, which the banks serve in one go)
                    const float4 q4 = *(const float4*)(q + (((i >> 2) * R + r) << 2)), k4 = *(const float4*)(k + (((i >> 2) * R + r) << 2));
                    qr[i] = q4.x; qr[i + 1] = q4.y; qr[i + 2] = q4.z; qr[i + 3] = q4.w;
                    kr[i] = k4.x; kr[i + 1] = k4.y; kr[i + 2] = k4.z; kr[i + 3] = k4.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    const int d = r + R * i;
                    qr[i] = d < D ? q[d] : 0.f;
                    kr[i] = d < D ? k[d] : (KIND == 1 ? 1.f : 0.f);      // a row that does not exist keeps its zero
                }
            }
            if (KIND == 0) {
                const float keep = gs[s * 4 + 2], take = gs[s * 4 + 3];
                const float tv = take * v;
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    S[i] = fmaf(keep, S[i], kr[i] * tv);
                    n[i] = fmaf(keep, n[i], take * kr[i]);
                    num = fmaf(S[i], qr[i], num);
                    nq = fmaf(n[i], qr[i], nq);
                }
            } else if (KIND == 2) {
                const float beta = gs[s * 4 + 0], decay = gs[s * 4 + 1];
                // (sums in up to four parts: one chain of DPT dependent multiply-adds would set the token's pace)
                constexpr int PARTS = DPT >= 4 ? 4 : 1;
                float part[PARTS];
#pragma unroll
                for (int j = 0; j < PARTS; ++j) part[j] = 0.f;
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    S[i] *= decay;
                    part[i % PARTS] = fmaf(S[i], kr[i], part[i % PARTS]);
                }
                float kS = PARTS == 4 ? (part[0] + part[1]) + (part[2] + part[3]) : part[0];
                // Two sums over a column's lanes a token: S^T k, which the update waits for, and the read-out, which
                // nothing waits for.  A warp issues in order, so the read-out's butterfly would hold up the next
                // token; it travels with the next token's first butterfly instead, and is stored a token late.
                float late = pending;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float other = __shfl_xor_sync(0xffffffffu, kS, o);
                    const float other_late = __shfl_xor_sync(0xffffffffu, late, o);
                    if (o < R) { kS += other; late += other_late; }
                }
                if (s > 0 && r == 0 && live) out_col[(size_t)(s0 + s - 1) * H * V] = late;
                const float u = beta * (v - kS);
#pragma unroll
                for (int j = 0; j < PARTS; ++j) part[j] = 0.f;
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    S[i] = fmaf(kr[i], u, S[i]);
                    part[i % PARTS] = fmaf(S[i], qr[i], part[i % PARTS]);
                }
                pending = PARTS == 4 ? (part[0] + part[1]) + (part[2] + part[3]) : part[0];
            } else if (KIND == 3) {
                const float keep = gs[s * 4 + 1];
                const float tv = gs[s * 4 + 0] * v;
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    S[i] = fmaf(keep, S[i], kr[i] * tv);
                    num = fmaf(S[i], qr[i], num);
                }
            } else {
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    const float f = kr[i];
                    S[i] = fmaf(f, S[i], (1.0f - f) * v);
                    num = fmaf(S[i], qr[i], num);
                }
            }
            if constexpr (KIND != 2) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {                // (R is a power of two; unrolled, the steps beyond it only pass)
                const float other = __shfl_xor_sync(0xffffffffu, num, o);
                if (o < R) num += other;
                if (KIND == 0) {
                    const float other_n = __shfl_xor_sync(0xffffffffu, nq, o);
                    if (o < R) nq += other_n;
                }
            }
            if (r == 0 && live) {
                float o = num;
                if (KIND == 0) o = num / (fmaxf(fabsf(nq), es[s]) + 1e-6f);
                if (KIND == 3 && a.d_skip) o = fmaf(a.d_skip[h], v, o);
                out_col[(size_t)(s0 + s) * H * V] = o;
            }
            }
        }
        if constexpr (KIND == 2) {                        // the chunk's last token's read-out
            float late = pending;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float other_late = __shfl_xor_sync(0xffffffffu, late, o);
                if (o < R) late += other_late;
            }
            if (r == 0 && live) out_col[(size_t)(s0 + ns - 1) * H * V] = late;
        }
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = FULL ? ((((i >> 2) * R + r) << 2) + (i & 3)) : r + R * i;
        if (d < D) {
            if (live) S_g[(size_t)d * V + col] = S[i];
            if (KIND == 0 && blockIdx.x == 0 && c == 0) a.nm_next[((size_t)b * H + h) * (D + 1) + d] = n[i];
        }
    }
    if (KIND == 0 && blockIdx.x == 0 && threadIdx.x == 0) a.nm_next[((size_t)b * H + h) * (D + 1) + D] = m;
}

__global__ void __launch_bounds__(128)
memory_commit_kernel(MemoryScanArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.y, h = blockIdx.x, H = a.H, D = a.D;
    float* srow = a.state + (size_t)a.seq_slot[b] * a.state_stride + (size_t)H * D * a.V;
    const float* src = a.nm_next + ((size_t)b * H + h) * (D + 1);
    for (int d = threadIdx.x; d < D; d += blockDim.x) srow[(size_t)h * D + d] = src[d];
    if (threadIdx.x == 0) srow[(size_t)H * D + h] = src[D];
}

template <typename TA, int DPT>
static int launch_memory_scan(const MemoryScanArgs& a, cudaStream_t stream) {
    int R = 1;
    while (R * DPT < a.D) R <<= 1;
    if (R > 32) return GL_ERR_SHAPE;
    const int CT = MS_THREADS / R;
    // tokens staged at a time: as many as 40 KB hold, at most 32 (a chunk costs a round trip to memory and
    // three block-wide waits, which a few tokens do not pay for)
    const int per_token = (2 * a.D + CT + 5) * (int)sizeof(float);
    int CH = (40 * 1024) / per_token;
    CH = CH > 32 ? 32 : CH;
    if (CH < 1) return GL_ERR_SMEM;
    const size_t smem = (size_t)CH * per_token;
    const dim3 grid((a.V + CT - 1) / CT, a.H, a.B);
    const bool full = DPT >= 4 && a.D == R * DPT;
    if (a.kind == 0) {
        if (full) return gl_launch_in_order(memory_scan_kernel<TA, DPT, 0, true>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
        return gl_launch_in_order(memory_scan_kernel<TA, DPT, 0, false>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
    }
    if (a.kind == 2) {
        if (full) return gl_launch_in_order(memory_scan_kernel<TA, DPT, 2, true>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
        return gl_launch_in_order(memory_scan_kernel<TA, DPT, 2, false>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
    }
    if (a.kind == 3) {
        if (full) return gl_launch_in_order(memory_scan_kernel<TA, DPT, 3, true>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
        return gl_launch_in_order(memory_scan_kernel<TA, DPT, 3, false>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
    }
    if (full) return gl_launch_in_order(memory_scan_kernel<TA, DPT, 1, true>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
    return gl_launch_in_order(memory_scan_kernel<TA, DPT, 1, false>, grid, dim3(MS_THREADS), smem, stream, a, R, CH);
}

static int memory_scan_blocks(const MemoryScanArgs& a, int dpt) {
    int R = 1;
    while (R * dpt < a.D) R <<= 1;
    if (R > 32) return -1;
    const int CT = MS_THREADS / R;
    return ((a.V + CT - 1) / CT) * a.H * a.B;
}

template <typename TA>
static int dispatch_memory_scan(const MemoryScanArgs& a, cudaStream_t stream) {
    // A thread walks the run's tokens one after the other, so the time of a long run is set by how little
    // each thread does per token and by how many warps an SM has to switch between: rows of a column are
    // spread over more lanes (fewer rows a thread) until the grid gives every SM several blocks.  With many
    // sequences of one token the widest threads do, and fewer blocks re-read the tokens' q and k.
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    // (the delta rule's token is a longer chain of dependent steps, which more rows a thread shorten: measured,
    // a grid of about one block an SM is its best, four an SM the other kinds')
    const int want = a.kind == 2 ? sms * 85 / 100 : 4 * sms;
    const int dpts[5] = {32, 8, 4, 2, 1};
    int pick = -1;
    for (int i = 0; i < 5; ++i) {
        const int blocks = memory_scan_blocks(a, dpts[i]);
        if (blocks < 0) continue;
        pick = dpts[i];                                  // the last that exists if none gives enough blocks
        if (blocks >= want) break;
    }
    if (a.rows_per_thread > 0 && memory_scan_blocks(a, a.rows_per_thread) > 0) pick = a.rows_per_thread;
    int rc;
    switch (pick) {
        case 32: rc = launch_memory_scan<TA, 32>(a, stream); break;
        case 8: rc = launch_memory_scan<TA, 8>(a, stream); break;
        case 4: rc = launch_memory_scan<TA, 4>(a, stream); break;
        case 2: rc = launch_memory_scan<TA, 2>(a, stream); break;
        case 1: rc = launch_memory_scan<TA, 1>(a, stream); break;
        default: return GL_ERR_SHAPE;
    }
    if (rc != 0 || a.kind != 0) return rc;
    return gl_launch(memory_commit_kernel, dim3(a.H, a.B), dim3(128), 0, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

GL_API int gl_memory_scan(const MemoryScanArgs* args, int act_dtype, cudaStream_t stream) {
    const MemoryScanArgs& a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.H <= 0 || a.D <= 0 || a.V <= 0 || a.D > 512 || a.B > 65535 || a.H > 65535) return GL_ERR_SHAPE;
    if (a.kind < 0 || a.kind > 3) return GL_ERR_SHAPE;
    if (a.kind == 2 && (!a.gates || !a.a_log || !a.dt_bias || a.KVH <= 0 || a.H % a.KVH)) return GL_ERR_SHAPE;
    if (a.kind == 3) {
        if (a.KVH <= 0 || a.H % a.KVH) return GL_ERR_SHAPE;
        if (a.gates ? (!a.a_log || !a.dt_bias) : !a.lower) return GL_ERR_SHAPE;
        if (a.cosv && (!a.sinv || a.rot_half <= 0 || 2 * a.rot_half > a.D)) return GL_ERR_SHAPE;
    }
    if (a.kind == 0 && (!(a.cap > 0.f) || !a.nm_next)) return GL_ERR_SHAPE;
    if (a.state_stride < (long long)a.H * a.D * a.V + (a.kind == 0 ? (long long)a.H * (a.D + 1) : 0)) return GL_ERR_SHAPE;
    if (act_dtype == GL_F32) return dispatch_memory_scan<float>(a, stream);
    if (act_dtype == GL_BF16) return dispatch_memory_scan<__nv_bfloat16>(a, stream);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Per-head unit norm of a memory's output, a weight and an optional gate:
//   out[t, h, j] = o[t, h, j] / sqrt(mean_j o[t, h, :]^2 + eps) * w * sigmoid(gate[t, h*V + j])
// w is [H*V] (w_per_head = 1) or [V] shared by the heads (null: no weight); gate (activation type, row pitch
// gate_ld, first column gate_off) may be absent; gate_silu multiplies by silu(gate) instead of the sigmoid.
// gate_first: gating first, then the norm of the gated values: out = g / sqrt(mean_j g^2 + eps) * w with g = o * act(gate).
// One warp per (token, head).
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* o, const float* __restrict__ w, const TA* gate, TA* __restrict__ out,
                      long long items, int H, int V, int w_per_head, int gate_ld, int gate_off, float eps, int gate_silu,
                      int gate_first) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const long long t = item / H;
    const int h = (int)(item - t * H);
    const float* src = o + (size_t)item * V;
    const TA* grow = gate ? gate + (size_t)t * gate_ld + gate_off + h * V : nullptr;
    const bool early = gate && gate_first;
    float q = 0.f;
    for (int j = lane; j < V; j += 32) {
        float v = src[j];
        if (early) { const float z = gl_load(grow + j); v *= gate_silu ? rc_silu(z) : rc_sigmoid(z); }
        q += v * v;
    }
    const float inv = 1.0f / sqrtf(gl_warp_sum(q) / (float)V + eps);
    for (int j = lane; j < V; j += 32) {
        float y = src[j];
        if (early) { const float z = gl_load(grow + j); y *= gate_silu ? rc_silu(z) : rc_sigmoid(z); }
        y *= inv;
        if (w) y *= w[w_per_head ? h * V + j : j];
        if (gate && !early) {
            const float z = gl_load(grow + j);
            y *= gate_silu ? rc_silu(z) : rc_sigmoid(z);
        }
        gl_store(out + (size_t)item * V + j, y);
    }
}

GL_API int gl_head_norm_gate(const float* o, const float* w, const void* gate, void* out, int T, int H, int V,
                             int w_per_head, int gate_ld, int gate_off, float eps, int act_dtype, int gate_silu,
                             int gate_first, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (H <= 0 || V <= 0) return GL_ERR_SHAPE;
    const long long items = (long long)T * H;
    const dim3 grid((unsigned)((items + 3) / 4));
    if (act_dtype == GL_F32)
        return gl_launch(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, 1, o, w, (const float*)gate, (float*)out,
                         items, H, V, w_per_head, gate_ld, gate_off, eps, gate_silu, gate_first);
    if (act_dtype == GL_BF16)
        return gl_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, o, w, (const __nv_bfloat16*)gate,
                         (__nv_bfloat16*)out, items, H, V, w_per_head, gate_ld, gate_off, eps, gate_silu, gate_first);
    return GL_ERR_DTYPE;
}

// 16 bytes of a row (4 floats or 8 bfloat16) as floats; both addresses 16-byte aligned
__device__ __forceinline__ void mc_load16(const float* src, float* dst) {
    *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
}
__device__ __forceinline__ void mc_load16(const __nv_bfloat16* src, float* dst) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
    const float2 f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
    reinterpret_cast<float4*>(dst)[0] = make_float4(f0.x, f0.y, f1.x, f1.y);
    reinterpret_cast<float4*>(dst)[1] = make_float4(f2.x, f2.y, f3.x, f3.y);
}

// 4 or 8 floats as 16 bytes of a row
__device__ __forceinline__ void mc_store16(float* dst, const float* v) {
    *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(v);
}
__device__ __forceinline__ void mc_store16(__nv_bfloat16* dst, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(v[0], v[1]);
    h[1] = __floats2bfloat162_rn(v[2], v[3]);
    h[2] = __floats2bfloat162_rn(v[4], v[5]);
    h[3] = __floats2bfloat162_rn(v[6], v[7]);
    *reinterpret_cast<uint4*>(dst) = raw;
}

// ---------------------------------------------------------------------------
// Short causal convolution per channel with bias and silu.  The filter's last tap is the current
// token's; inputs before the run come from the sequence's state row (the last taps-1 inputs, oldest
// first, zero at a sequence's start).  A second kernel then moves the run's last inputs into the row.
// ---------------------------------------------------------------------------
struct ConvArgs {
    const void* x;            // [T, ld] activation type; the convolved channels start at column x_off
    void* out;                // [T, C] activation type
    const float* w;           // [C, taps]
    const float* bias;        // [C] or null
    float* state;             // [slots, state_stride]; the tail [C, taps-1] starts at tail_off
    const int* tok_seq;       // [T]
    const int* seq_slot;
    const int* seq_qstart;
    const int* seq_qlen;
    int T, B, C, taps, ld, x_off, state_stride, tail_off;
};

template <typename TA>
__global__ void __launch_bounds__(256)
conv_silu_kernel(ConvArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.T * a.C) return;
    const int t = (int)(i / a.C), c = (int)(i - (long long)t * a.C);
    const int b = a.tok_seq[t];
    const int idx = t - a.seq_qstart[b];
    const int back = a.taps - 1;
    const float* tail = a.state + (size_t)a.seq_slot[b] * a.state_stride + a.tail_off + (size_t)c * back;
    float acc = a.bias ? a.bias[c] : 0.f;
    for (int j = 0; j < a.taps; ++j) {
        const int rel = idx - back + j;               // place in the run; negative: before it
        const float v = rel >= 0 ? gl_load((const TA*)a.x + (size_t)(t - back + j) * a.ld + a.x_off + c) : tail[rel + back];
        acc = fmaf(a.w[(size_t)c * a.taps + j], v, acc);
    }
    gl_store((TA*)a.out + (size_t)t * a.C + c, rc_silu(acc));
}

// The same with 16 bytes of channels a thread (4 or 8 of them): columns, pitch and offset are whole pieces, and
// the thread's TAPS x channels weights are one run of memory that it fetches 16 bytes at a time.  The sums run in
// the order of the kernel above.
template <typename TA, int TAPS>
__global__ void __launch_bounds__(256)
conv_silu_wide_kernel(ConvArgs a) {
    constexpr int VEC = 16 / (int)sizeof(TA);
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int CV = a.C / VEC;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.T * CV) return;
    const int t = (int)(i / CV), c0 = (int)(i - (long long)t * CV) * VEC;
    const int b = a.tok_seq[t];
    const int idx = t - a.seq_qstart[b];
    constexpr int back = TAPS - 1;
    const float* tail = a.state + (size_t)a.seq_slot[b] * a.state_stride + a.tail_off;
    __align__(16) float acc[VEC], v[VEC], w[VEC * TAPS];
#pragma unroll
    for (int q = 0; q < VEC * TAPS / 4; ++q)
        reinterpret_cast<float4*>(w)[q] = reinterpret_cast<const float4*>(a.w + (size_t)c0 * TAPS)[q];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = a.bias ? a.bias[c0 + k] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
        const int rel = idx - back + j;               // place in the run; negative: before it
        if (rel >= 0) {
            mc_load16((const TA*)a.x + (size_t)(t - back + j) * a.ld + a.x_off + c0, v);
        } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[k] = tail[(size_t)(c0 + k) * back + rel + back];
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = fmaf(w[k * TAPS + j], v[k], acc[k]);
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = rc_silu(acc[k]);
    mc_store16((TA*)a.out + (size_t)t * a.C + c0, acc);
}

template <typename TA>
static int launch_conv_silu_wide(const ConvArgs& a, dim3 grid, cudaStream_t stream) {
    switch (a.taps) {
        case 1: return gl_launch(conv_silu_wide_kernel<TA, 1>, grid, dim3(256), 0, stream, 1, a);
        case 2: return gl_launch(conv_silu_wide_kernel<TA, 2>, grid, dim3(256), 0, stream, 1, a);
        case 3: return gl_launch(conv_silu_wide_kernel<TA, 3>, grid, dim3(256), 0, stream, 1, a);
        default: return gl_launch(conv_silu_wide_kernel<TA, 4>, grid, dim3(256), 0, stream, 1, a);
    }
}

template <typename TA>
__global__ void __launch_bounds__(256)
conv_tail_kernel(ConvArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.B * a.C) return;
    const int b = (int)(i / a.C), c = (int)(i - (long long)b * a.C);
    const int back = a.taps - 1, qlen = a.seq_qlen[b], qstart = a.seq_qstart[b];
    float* tail = a.state + (size_t)a.seq_slot[b] * a.state_stride + a.tail_off + (size_t)c * back;
    for (int k = 0; k < back; ++k) {                  // ascending: a place is read before a lower one is written
        const int rel = qlen - back + k;
        tail[k] = rel >= 0 ? gl_load((const TA*)a.x + (size_t)(qstart + rel) * a.ld + a.x_off + c) : tail[qlen + k];
    }
}

// One token a sequence: a thread owns a (sequence, channel), so it may read the tail, write the output and
// shift the tail in one go.
template <typename TA>
__global__ void __launch_bounds__(256)
conv_silu_step_kernel(ConvArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.B * a.C) return;
    const int b = (int)(i / a.C), c = (int)(i - (long long)b * a.C);
    const int back = a.taps - 1, t = a.seq_qstart[b];
    float* tail = a.state + (size_t)a.seq_slot[b] * a.state_stride + a.tail_off + (size_t)c * back;
    const float x = gl_load((const TA*)a.x + (size_t)t * a.ld + a.x_off + c);
    float acc = a.bias ? a.bias[c] : 0.f;
    for (int j = 0; j < back; ++j) {
        const float v = tail[j];
        acc = fmaf(a.w[(size_t)c * a.taps + j], v, acc);
        if (j > 0) tail[j - 1] = v;                   // (read before the place below it is written)
    }
    acc = fmaf(a.w[(size_t)c * a.taps + back], x, acc);
    if (back > 0) tail[back - 1] = x;
    gl_store((TA*)a.out + (size_t)t * a.C + c, rc_silu(acc));
}

GL_API int gl_conv_silu(const ConvArgs* args, int act_dtype, cudaStream_t stream) {
    const ConvArgs& a = *args;
    if (a.T <= 0 || a.B <= 0) return GL_OK;
    if (a.C <= 0 || a.taps <= 0) return GL_ERR_SHAPE;
    const long long n = (long long)a.T * a.C, nb = (long long)a.B * a.C;
    const dim3 g1((unsigned)((n + 255) / 256)), g2((unsigned)((nb + 255) / 256));
    int rc;
    if (a.T == a.B) {                                 // every sequence brings exactly one token
        if (act_dtype == GL_F32) return gl_launch(conv_silu_step_kernel<float>, g2, dim3(256), 0, stream, 1, a);
        if (act_dtype == GL_BF16) return gl_launch(conv_silu_step_kernel<__nv_bfloat16>, g2, dim3(256), 0, stream, 1, a);
        return GL_ERR_DTYPE;
    }
    // rows of whole, aligned 16-byte pieces: a thread takes a piece of channels
    const int vec = act_dtype == GL_F32 ? 4 : 8;
    const bool wide = a.taps <= 4 && ((size_t)a.w & 15) == 0 && a.C % vec == 0 && a.ld % vec == 0 && a.x_off % vec == 0 && ((size_t)a.x & 15) == 0 && ((size_t)a.out & 15) == 0;
    const dim3 gw((unsigned)((n / vec + 255) / 256));
    if (act_dtype == GL_F32) {
        rc = wide ? launch_conv_silu_wide<float>(a, gw, stream)
                  : gl_launch(conv_silu_kernel<float>, g1, dim3(256), 0, stream, 1, a);
        if (rc == 0 && a.taps > 1) rc = gl_launch(conv_tail_kernel<float>, g2, dim3(256), 0, stream, 1, a);
        return rc;
    }
    if (act_dtype == GL_BF16) {
        rc = wide ? launch_conv_silu_wide<__nv_bfloat16>(a, gw, stream)
                  : gl_launch(conv_silu_kernel<__nv_bfloat16>, g1, dim3(256), 0, stream, 1, a);
        if (rc == 0 && a.taps > 1) rc = gl_launch(conv_tail_kernel<__nv_bfloat16>, g2, dim3(256), 0, stream, 1, a);
        return rc;
    }
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Selective scan.  Per channel c and state n:
//   dt = softplus(dtp[t, c]);  S[c, n] <- e^(dt A[c, n]) S[c, n] + dt x[t, c] B[t, n],  A = -e^(A_log)
//   y[t, c] = (sum_n S[c, n] C[t, n] + D[c] x[t, c]) * silu(z[t, c])
// A channel's states are spread over G adjacent lanes, NPT states a lane (fewer states a lane and more lanes
// when the grid would otherwise leave the SMs with a warp or two each: a thread walks the tokens in order).
// ---------------------------------------------------------------------------
struct SelectiveScanArgs {
    const void* x;            // [T, C] activation type (the convolution's output)
    const float* dtp;         // [T, C] 32-bit: the step size before softplus, bias included
    const void* bc;           // [T, 2N] activation type: B then C
    const void* z;            // activation type, row pitch z_ld, first column z_off
    void* out;                // [T, C] activation type
    const float* a_log;       // [C, N]
    const float* d_skip;      // [C]
    float* state;             // [slots, state_stride], S [C, N] first
    const int* seq_slot;
    const int* seq_qstart;
    const int* seq_qlen;
    int B, C, N, z_ld, z_off, state_stride;
    // a long run cut into chunks of chunk_len tokens that are walked side by side (n_chunks > 1):
    //   first every chunk from a zero state, keeping its last state and the sum of its step sizes;
    //   then a carry over the chunks, S_start[k+1] = e^(A sum_k) S_start[k] + last_k (the decays of a chunk
    //   multiply to e^(A sum of its step sizes));  then every chunk again from its true start, with outputs.
    float* chunk_state;       // [B, n_chunks, C, N]
    float* chunk_dt;          // [B, n_chunks, C]
    int chunk_len, n_chunks;
};

// MODE 0: a run in one piece.  MODE 1: a chunk from a zero state, no outputs.  MODE 2: a chunk from its start.
template <typename TA, int SS_NPT, int MODE>
__global__ void __launch_bounds__(RC_THREADS)
selective_scan_kernel(SelectiveScanArgs a, int G) {
    extern __shared__ float smem[];
    // (launched in order, not early: placed beside the kernel before, the blocks of a scan sat several to an SM
    // for its whole length, and a prompt of 2,048 tokens took 25 ms instead of 16)
    gl_grid_wait();
    const int N = a.N, C = a.C;
    const int CPB = RC_THREADS / G;
    const int b = blockIdx.y, c0 = blockIdx.x * CPB;
    const int g = threadIdx.x % G, cl = threadIdx.x / G;
    const int c = c0 + cl;
    const bool live = c < C;
    const int qlen = a.seq_qlen[b], qstart = a.seq_qstart[b];
    const int chunk = MODE == 0 ? 0 : blockIdx.z;
    const int t_begin = MODE == 0 ? 0 : chunk * a.chunk_len;
    const int t_end = MODE == 0 ? qlen : min(qlen, t_begin + a.chunk_len);
    if (t_begin >= qlen) return;                      // (the whole block: this sequence has no such chunk)
    float* Bs = smem;                                 // [CHUNK][N]
    float* Cs = Bs + SS_CHUNK * N;                    // [CHUNK][N]
    float* ds = Cs + SS_CHUNK * N;                    // [CHUNK][CPB] step sizes
    float* xs = ds + SS_CHUNK * CPB;                  // [CHUNK][CPB]
    float* zs = xs + SS_CHUNK * CPB;                  // [CHUNK][CPB]
    float* S_g = a.state + (size_t)a.seq_slot[b] * a.state_stride + (size_t)(live ? c : 0) * N;
    float* S_c = MODE == 0 ? S_g : a.chunk_state + (((size_t)b * a.n_chunks + chunk) * C + (live ? c : 0)) * N;
    float S[SS_NPT], A[SS_NPT];
#pragma unroll
    for (int i = 0; i < SS_NPT; ++i) {
        const int n = g + G * i;
        const bool ok = live && n < N;
        S[i] = (ok && MODE != 1) ? (MODE == 0 ? S_g[n] : S_c[n]) : 0.f;
        A[i] = ok ? -expf(a.a_log[(size_t)c * N + n]) : 0.f;
    }
    float dt_sum = 0.f;
    for (int s0 = t_begin; s0 < t_end; s0 += SS_CHUNK) {
        const int ns = min(SS_CHUNK, t_end - s0);
        __syncthreads();
        for (int e = threadIdx.x; e < ns * N; e += RC_THREADS) {
            const int s = e / N, n = e - s * N;
            const TA* row = (const TA*)a.bc + (size_t)(qstart + s0 + s) * 2 * N;
            Bs[e] = gl_load(row + n);
            Cs[e] = gl_load(row + N + n);
        }
        for (int e = threadIdx.x; e < ns * CPB; e += RC_THREADS) {
            const int s = e / CPB, j = e - s * CPB;
            const size_t t = (size_t)(qstart + s0 + s);
            const bool ok = c0 + j < C;
            ds[e] = ok ? rc_softplus(a.dtp[t * C + c0 + j]) : 0.f;
            xs[e] = ok ? gl_load((const TA*)a.x + t * C + c0 + j) : 0.f;
            zs[e] = ok ? gl_load((const TA*)a.z + t * a.z_ld + a.z_off + c0 + j) : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int s = 0; s < ns; ++s) {
            const float dt = ds[s * CPB + cl], x = xs[s * CPB + cl];
            const float dx = dt * x;
            if (MODE == 1) dt_sum += dt;
            const float* Bt = Bs + s * N;
            const float* Ct = Cs + s * N;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < SS_NPT; ++i) {
                const int n = g + G * i;
                if (n < N) {
                    S[i] = fmaf(rc_decay(dt * A[i]), S[i], dx * Bt[n]);
                    y = fmaf(S[i], Ct[n], y);
                }
            }
            for (int o = G >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (g == 0) ds[s * CPB + cl] = y;           // the step size has been used: its place takes the sum
        }
        if (MODE == 1) continue;
        __syncthreads();
        // the skip connection and the gate do not go from token to token: all of the chunk's outputs at once
        for (int e = threadIdx.x; e < ns * CPB; e += RC_THREADS) {
            const int s = e / CPB, j = e - s * CPB;
            if (c0 + j < C) {
                const float y = fmaf(a.d_skip[c0 + j], xs[e], ds[e]);
                gl_store((TA*)a.out + (size_t)(qstart + s0 + s) * C + c0 + j, y * rc_silu(zs[e]));
            }
        }
    }
    if (live && (MODE != 2 || t_end == qlen)) {       // the state row takes the run's last state
        float* dst = MODE == 1 ? S_c : S_g;
#pragma unroll
        for (int i = 0; i < SS_NPT; ++i) {
            const int n = g + G * i;
            if (n < N) dst[n] = S[i];
        }
    }
    if (MODE == 1 && live && g == 0) a.chunk_dt[((size_t)b * a.n_chunks + chunk) * C + c] = dt_sum;
}

// Between the two walks: every chunk's start state from the run's start state and the chunks' last states.
__global__ void __launch_bounds__(128)
selective_carry_kernel(SelectiveScanArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.y;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.C * a.N) return;
    const int c = (int)(i / a.N);
    const int chunks = (a.seq_qlen[b] + a.chunk_len - 1) / a.chunk_len;
    float S = a.state[(size_t)a.seq_slot[b] * a.state_stride + i];
    const float A = -expf(a.a_log[i]);
    for (int k = 0; k < chunks; ++k) {
        float* slot = a.chunk_state + ((size_t)b * a.n_chunks + k) * a.C * a.N + i;
        const float last = *slot;
        *slot = S;
        S = fmaf(expf(A * a.chunk_dt[((size_t)b * a.n_chunks + k) * a.C + c]), S, last);
    }
}

template <typename TA, int NPT>
static int launch_selective_scan(const SelectiveScanArgs& a, cudaStream_t stream) {
    int G = 1;
    while (G * NPT < a.N) G <<= 1;
    if (G > 32) return GL_ERR_SHAPE;
    const int CPB = RC_THREADS / G;
    const size_t smem = (size_t)SS_CHUNK * (2 * a.N + 3 * CPB) * sizeof(float);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    if (a.n_chunks <= 1) {
        const dim3 grid((a.C + CPB - 1) / CPB, a.B);
        return gl_launch_in_order(selective_scan_kernel<TA, NPT, 0>, grid, dim3(RC_THREADS), smem, stream, a, G);
    }
    const dim3 grid((a.C + CPB - 1) / CPB, a.B, a.n_chunks);
    int rc = gl_launch_in_order(selective_scan_kernel<TA, NPT, 1>, grid, dim3(RC_THREADS), smem, stream, a, G);
    if (rc != 0) return rc;
    const long long n = (long long)a.C * a.N;
    rc = gl_launch(selective_carry_kernel, dim3((unsigned)((n + 127) / 128), a.B), dim3(128), 0, stream, 1, a);
    if (rc != 0) return rc;
    return gl_launch_in_order(selective_scan_kernel<TA, NPT, 2>, grid, dim3(RC_THREADS), smem, stream, a, G);
}

static int selective_scan_blocks(const SelectiveScanArgs& a, int npt) {
    int G = 1;
    while (G * npt < a.N) G <<= 1;
    if (G > 32) return -1;
    const int CPB = RC_THREADS / G;
    return ((a.C + CPB - 1) / CPB) * a.B * (a.n_chunks > 1 ? a.n_chunks : 1);
}

template <typename TA>
static int dispatch_selective_scan(const SelectiveScanArgs& a, cudaStream_t stream) {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int want = 4 * sms;
    const int b8 = selective_scan_blocks(a, 8), b2 = selective_scan_blocks(a, 2), b1 = selective_scan_blocks(a, 1);
    if (b8 >= want || (b2 < 0 && b1 < 0)) return launch_selective_scan<TA, 8>(a, stream);
    if (b2 >= want || b1 < 0) return b2 >= 0 ? launch_selective_scan<TA, 2>(a, stream) : launch_selective_scan<TA, 8>(a, stream);
    return launch_selective_scan<TA, 1>(a, stream);
}

GL_API int gl_selective_scan(const SelectiveScanArgs* args, int act_dtype, cudaStream_t stream) {
    const SelectiveScanArgs& a = *args;
    if (a.B <= 0) return GL_OK;
    if (a.C <= 0 || a.N <= 0 || a.N > 256 || a.B > 65535) return GL_ERR_SHAPE;
    if (a.n_chunks > 1 && (!a.chunk_state || !a.chunk_dt || a.chunk_len <= 0 || a.n_chunks > 65535)) return GL_ERR_SHAPE;
    if (act_dtype == GL_F32) return dispatch_selective_scan<float>(a, stream);
    if (act_dtype == GL_BF16) return dispatch_selective_scan<__nv_bfloat16>(a, stream);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// The matrix memories for long runs: chunks of tokens side by side, a lane a column.
//
// Written with a decay a_t[d] and an input b_t[d] per row (gated kind: a = keep_t for every row, b = take_t
// k_t[d]; bounded forget: a = f_t[d], b = 1 - f_t[d]) a memory is S' = diag(a) S + b v^T, column by column.
// A thread owns one column and keeps all of its rows in registers: a token costs it two multiply-adds a row
// and nothing is exchanged between lanes.  The gated kind's normaliser n is one more column whose value is
// always 1 (its "output" is n.q), so it needs no code of its own.  That mapping has only heads x columns / 32
// warps of work, so a run is cut into chunks that are walked side by side, twice:
//   walk 1: every chunk from a zero state; its last state goes to chunk_state;
//   carry:  S_start[k+1] = diag(P_k) S_start[k] + last_k, P_k[d] the product of the chunk's decays;
//   walk 2: every chunk from its start, with the raw outputs S^T q (the gated kind's division by
//           max(|n.q|, e^-m) + 1e-6 follows as a pass of its own over all tokens at once).
// The gated kind's gates come from a pass of their own: the log gates of all tokens side by side, then the
// running maximum token by token (a thread a head), which leaves keep, take and e^-m per token.
// The plain decay (kind 3) is the gated kind without a normaliser: keep and take per (token, head) come from a pass
// of their own (a fixed decay, or a step size: the formulas of memory_scan_kernel), a = keep for every row,
// b = k after its rotation and scale, and the token's value is multiplied by take before it enters, so that a
// chunk's arithmetic is the token-by-token kernel's.  q and k heads may be shared by several heads; the skip
// term d_skip[h] v is added to the read-out.
// ---------------------------------------------------------------------------
struct MemoryChunkArgs {
    const void* proj;         // [T, ld] activation type
    float* out;               // [T, H*V] raw S^T q
    float* nq;                // gated: [T, H] n.q
    float* gates;             // gated: [T, H, 4]: log input gate, log forget gate -> keep, take, e^-m, unused
    float* state;             // [slots, state_stride]: S [H, D, V], gated: n [H, D], m [H]
    const float* lower;       // bounded forget: [H*D]
    float* chunk_state;       // [B, n_chunks, H, D, cols]
    float* chunk_decay;       // [B, n_chunks, H, D]
    const int* tok_seq;       // [T]
    const int* seq_slot;
    const int* seq_qstart;
    const int* seq_qlen;
    int T, ld, q_off, k_off, v_off, i_off, f_off;
    int B, H, D, V, cols, state_stride, kind, chunk_len, n_chunks;
    float cap, q_scale;
    // kind 3:
    const void* gates_in;     // [T, gates_ld] activation type or null: the step sizes' projections (column f_off + h)
    const float* a_log;       // [H]
    const float* dt_bias;     // [H]
    const float* cosv;        // [T, rot_half] or null
    const float* sinv;
    const float* d_skip;      // [H] or null
    int gates_ld, KVH, rot_half;
    float k_scale;
};

#define MC_THREADS 128
#define MC_TOKENS 16

// log gates of every token: gates[t, h, 0] = cap tanh(i / cap), gates[t, h, 1] = logsigmoid(cap tanh(f / cap))
template <typename TA>
__global__ void __launch_bounds__(256)
memory_log_gates_kernel(MemoryChunkArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.T * a.H) return;
    const int t = (int)(i / a.H), h = (int)(i - (long long)t * a.H);
    const TA* row = (const TA*)a.proj + (size_t)t * a.ld;
    a.gates[i * 4 + 0] = a.cap * tanhf(gl_load(row + a.i_off + h) / a.cap);
    a.gates[i * 4 + 1] = rc_log_sigmoid(a.cap * tanhf(gl_load(row + a.f_off + h) / a.cap));
}

// the running maximum, token by token, a warp a (sequence, head): 32 tokens' log gates are fetched at once, the
// maximum walks them in registers (every lane follows it, lane j keeps token j's), and the lanes then take
// keep, take and e^-m of their tokens side by side
__global__ void __launch_bounds__(32)
memory_gate_walk_kernel(MemoryChunkArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.x / a.H, h = blockIdx.x - b * a.H, lane = threadIdx.x;
    float* m_g = a.state + (size_t)a.seq_slot[b] * a.state_stride + (size_t)a.H * a.D * a.V + (size_t)a.H * a.D + h;
    float m = *m_g;
    const int qstart = a.seq_qstart[b], qlen = a.seq_qlen[b];
    for (int s0 = 0; s0 < qlen; s0 += 32) {
        const bool ok = s0 + lane < qlen;
        float* g = a.gates + ((size_t)(qstart + s0 + (ok ? lane : 0)) * a.H + h) * 4;
        const float gi = ok ? g[0] : -INFINITY, gf = ok ? g[1] : 0.f;      // a token that is not there leaves m as it is
        float m_old = 0.f, m_mine = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float m_new = fmaxf(__shfl_sync(0xffffffffu, gf, j) + m, __shfl_sync(0xffffffffu, gi, j));
            if (lane == j) { m_old = m; m_mine = m_new; }
            m = m_new;
        }
        if (ok) {
            g[0] = rc_decay(gf + m_old - m_mine);
            g[1] = expf(gi - m_mine);
            g[2] = expf(-m_mine);
        }
    }
    if (lane == 0) *m_g = m;
}

// the plain decay's keep and take of every token: gates[t, h, 0] = keep, gates[t, h, 1] = take
template <typename TA>
__global__ void __launch_bounds__(256)
memory_decay_gates_kernel(MemoryChunkArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.T * a.H) return;
    const int t = (int)(i / a.H), h = (int)(i - (long long)t * a.H);
    float take = 1.0f, keep = a.lower ? a.lower[h] : 1.0f;
    if (a.gates_in) {
        take = rc_softplus(gl_load((const TA*)a.gates_in + (size_t)t * a.gates_ld + a.f_off + h) + a.dt_bias[h]);
        keep = rc_decay(-expf(a.a_log[h]) * take);
    }
    a.gates[i * 4 + 0] = keep;
    a.gates[i * 4 + 1] = take;
}

// the product of a chunk's decays per row
template <typename TA, int KIND>
__global__ void __launch_bounds__(128)
memory_chunk_decay_kernel(MemoryChunkArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.z / a.n_chunks, chunk = blockIdx.z - b * a.n_chunks, h = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    const int qlen = a.seq_qlen[b], qstart = a.seq_qstart[b];
    const int t0 = chunk * a.chunk_len, t1 = min(qlen, t0 + a.chunk_len);
    if (d >= a.D || t0 >= qlen) return;
    float p = 1.0f;
    const float l = KIND == 1 ? a.lower[h * a.D + d] : 0.f;
    for (int s = t0; s < t1; ++s) {
        if (KIND == 0 || KIND == 3) p *= a.gates[((size_t)(qstart + s) * a.H + h) * 4];
        else p *= l + (1.0f - l) * rc_sigmoid(gl_load((const TA*)a.proj + (size_t)(qstart + s) * a.ld + a.f_off + h * a.D + d));
    }
    a.chunk_decay[(((size_t)b * a.n_chunks + chunk) * a.H + h) * a.D + d] = p;
}

// two 32-bit multiply-adds in one instruction (the pair's halves are independent and rounded like fmaf's)
__device__ __forceinline__ unsigned long long mc_pack(float x, float y) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ unsigned long long mc_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long mc_mul2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float2 mc_unpack(unsigned long long v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}

// MODE 1: from zero, keep the last state.  MODE 2: from the chunk's start, with outputs.  NT: threads (columns) a block.
// FULL: D == DMAX, so no row needs a bounds check; a token's rows are then read four at a time and updated in
// pairs (fma.rn.f32x2), and the read-out is summed in four parts (the walk issues less than half the
// instructions a row that the checked form does, which is what bounds it).
template <typename TA, int DMAX, int KIND, int MODE, int NT, bool FULL>
__global__ void __launch_bounds__(NT)
memory_chunk_walk_kernel(MemoryChunkArgs a) {
    extern __shared__ __align__(16) float smem[];
    gl_grid_wait();
    const int D = a.D, V = a.V, H = a.H, cols = a.cols;
    const int b = blockIdx.z / a.n_chunks, chunk = blockIdx.z - b * a.n_chunks, h = blockIdx.y;
    const int col0 = blockIdx.x * NT, col = col0 + threadIdx.x;
    const bool live = col < cols;
    const int qlen = a.seq_qlen[b], qstart = a.seq_qstart[b];
    const int t0 = chunk * a.chunk_len, t1 = min(qlen, t0 + a.chunk_len);
    if (t0 >= qlen) return;
    constexpr bool SCALAR = KIND == 0 || KIND == 3;   // one decay for all rows of a (token, head)
    float* as = smem;                                 // [TOKENS][D] decay (bounded forget; the other kinds' is a scalar)
    float* bs = as + MC_TOKENS * D;                   // [TOKENS][D] input per row
    float* qs = bs + MC_TOKENS * D;                   // [TOKENS][D]
    float* vs = qs + MC_TOKENS * D;                   // [TOKENS][NT]
    float* ks = vs + MC_TOKENS * NT;                  // [TOKENS] the scalar keep
    float* ts = ks + MC_TOKENS;                       // [TOKENS] the plain decay's take
    const int kh = KIND == 3 ? h / (H / a.KVH) : h;   // the head of q and k this head reads
    constexpr int VEC = 16 / (int)sizeof(TA);
    // rows of whole, aligned 16-byte pieces can be fetched as such
    const bool wide = KIND == 3 && D % VEC == 0 && V % VEC == 0 && a.ld % VEC == 0 && a.q_off % VEC == 0
                      && a.k_off % VEC == 0 && a.v_off % VEC == 0 && ((size_t)a.proj & 15) == 0;
    float* cs = a.chunk_state + ((((size_t)b * a.n_chunks + chunk) * H + h) * D) * cols;
    float S[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (MODE == 2 && live && d < D) ? cs[(size_t)d * cols + col] : 0.f;
    for (int s0 = t0; s0 < t1; s0 += MC_TOKENS) {
        const int ns = min(MC_TOKENS, t1 - s0);
        __syncthreads();
        if (KIND == 3 && wide) {
            // whole 16-byte pieces of the rows first, as they are; then rotation and scale in place
            const int DV = D / VEC;
            for (int e = threadIdx.x; e < ns * DV; e += NT) {
                const int s = e / DV, d = (e - s * DV) * VEC;
                const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
                mc_load16(row + a.k_off + kh * D + d, bs + s * D + d);
                if (MODE == 2) mc_load16(row + a.q_off + kh * D + d, qs + s * D + d);
            }
            for (int e = threadIdx.x; e < ns * (NT / VEC); e += NT) {
                const int s = e / (NT / VEC), j = (e - s * (NT / VEC)) * VEC;
                const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
                if (col0 + j < V) mc_load16(row + a.v_off + h * V + col0 + j, vs + s * NT + j);   // (V is whole pieces)
            }
            if (a.cosv || a.k_scale != 1.0f || (MODE == 2 && a.q_scale != 1.0f)) {
                __syncthreads();
                const int half = a.cosv ? a.rot_half : 0;
                for (int e = threadIdx.x; e < ns * D; e += NT) {
                    const int s = e / D, d = e - s * D;
                    if (d < half) {
                        // the pair (u, v) = (dim d, dim d + half) becomes (u c - v s, v c + u s)
                        const size_t t = (size_t)(qstart + s0 + s);
                        const float c = a.cosv[t * half + d], sn = a.sinv[t * half + d];
                        const float ku = bs[e], kv = bs[e + half];
                        bs[e] = (ku * c - kv * sn) * a.k_scale;
                        bs[e + half] = (kv * c + ku * sn) * a.k_scale;
                        if (MODE == 2) {
                            const float qu = qs[e], qv = qs[e + half];
                            qs[e] = (qu * c - qv * sn) * a.q_scale;
                            qs[e + half] = (qv * c + qu * sn) * a.q_scale;
                        }
                    } else if (d >= 2 * half) {
                        bs[e] *= a.k_scale;
                        if (MODE == 2) qs[e] *= a.q_scale;
                    }
                }
            }
        } else {
#pragma unroll 4
            for (int e = threadIdx.x; e < ns * D; e += NT) {
                const int s = e / D, d = e - s * D;
                const size_t t = (size_t)(qstart + s0 + s);
                const TA* row = (const TA*)a.proj + t * a.ld;
                if (KIND == 0) {
                    bs[e] = a.gates[(t * H + h) * 4 + 1] * gl_load(row + a.k_off + h * D + d);
                    if (MODE == 2) qs[e] = gl_load(row + a.q_off + h * D + d) * a.q_scale;
                } else if (KIND == 3) {
                    float kv = gl_load(row + a.k_off + kh * D + d), qv = MODE == 2 ? gl_load(row + a.q_off + kh * D + d) : 0.f;
                    if (a.cosv && d < 2 * a.rot_half) {
                        // the pair (u, v) = (dim i, dim i + rot_half) becomes (u c - v s, v c + u s)
                        const bool first = d < a.rot_half;
                        const int i = first ? d : d - a.rot_half, other = first ? d + a.rot_half : d - a.rot_half;
                        const float c = a.cosv[t * a.rot_half + i], sn = a.sinv[t * a.rot_half + i];
                        const float ko = gl_load(row + a.k_off + kh * D + other);
                        kv = first ? kv * c - ko * sn : kv * c + ko * sn;
                        if (MODE == 2) {
                            const float qo = gl_load(row + a.q_off + kh * D + other);
                            qv = first ? qv * c - qo * sn : qv * c + qo * sn;
                        }
                    }
                    bs[e] = kv * a.k_scale;
                    if (MODE == 2) qs[e] = qv * a.q_scale;
                } else {
                    const float l = a.lower[h * D + d];
                    const float f = l + (1.0f - l) * rc_sigmoid(gl_load(row + a.f_off + h * D + d));
                    as[e] = f;
                    bs[e] = 1.0f - f;
                    if (MODE == 2) qs[e] = rc_silu(gl_load(row + a.q_off + h * D + d));
                }
            }
            for (int e = threadIdx.x; e < ns * NT; e += NT) {
                const int s = e / NT, j = col0 + (e - s * NT);
                const TA* row = (const TA*)a.proj + (size_t)(qstart + s0 + s) * a.ld;
                vs[e] = j < V ? gl_load(row + a.v_off + h * V + j) : 1.0f;     // the normaliser's column takes 1
            }
        }
        if (SCALAR && threadIdx.x < ns) {
            const float* g = a.gates + ((size_t)(qstart + s0 + threadIdx.x) * H + h) * 4;
            ks[threadIdx.x] = g[0];
            if (KIND == 3) ts[threadIdx.x] = g[1];
        }
        __syncthreads();
        for (int s = 0; s < ns; ++s) {
            const float v_in = vs[s * NT + threadIdx.x];
            const float v = KIND == 3 ? ts[s] * v_in : v_in;
            const float keep = SCALAR ? ks[s] : 0.f;
            const float* ar = as + s * D;
            const float* br = bs + s * D;
            const float* qr = qs + s * D;
            float num = 0.f;
            if constexpr (FULL) {
                const unsigned long long v2 = mc_pack(v, v), keep2 = mc_pack(keep, keep);
                unsigned long long n01 = mc_pack(0.f, 0.f), n23 = n01;
#pragma unroll
                for (int d = 0; d < DMAX; d += 4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(br + d);
                    unsigned long long a01 = keep2, a23 = keep2;
                    if (!SCALAR) {
                        const float4 a4 = *reinterpret_cast<const float4*>(ar + d);
                        a01 = mc_pack(a4.x, a4.y);
                        a23 = mc_pack(a4.z, a4.w);
                    }
                    unsigned long long s01 = mc_pack(S[d], S[d + 1]), s23 = mc_pack(S[d + 2], S[d + 3]);
                    s01 = mc_fma2(a01, s01, mc_mul2(mc_pack(b4.x, b4.y), v2));
                    s23 = mc_fma2(a23, s23, mc_mul2(mc_pack(b4.z, b4.w), v2));
                    if (MODE == 2) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qr + d);
                        n01 = mc_fma2(s01, mc_pack(q4.x, q4.y), n01);
                        n23 = mc_fma2(s23, mc_pack(q4.z, q4.w), n23);
                    }
                    const float2 r01 = mc_unpack(s01), r23 = mc_unpack(s23);
                    S[d] = r01.x; S[d + 1] = r01.y; S[d + 2] = r23.x; S[d + 3] = r23.y;
                }
                if (MODE == 2) {
                    const float2 p01 = mc_unpack(n01), p23 = mc_unpack(n23);
                    num = (p01.x + p01.y) + (p23.x + p23.y);
                }
            } else {
#pragma unroll
                for (int d = 0; d < DMAX; ++d) {
                    if (d < D) {
                        S[d] = fmaf(SCALAR ? keep : ar[d], S[d], br[d] * v);
                        if (MODE == 2) num = fmaf(S[d], qr[d], num);
                    }
                }
            }
            if (MODE == 2 && live) {
                const size_t t = (size_t)(qstart + s0 + s);
                if (KIND == 3 && a.d_skip) num = fmaf(a.d_skip[h], v_in, num);
                if (col < V) a.out[t * H * V + (size_t)h * V + col] = num;
                else a.nq[t * H + h] = num;
            }
        }
    }
    if (!live) return;
    if (MODE == 1) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
            if (d < D) cs[(size_t)d * cols + col] = S[d];
    } else if (t1 == qlen) {                          // the run's last chunk: the state row takes its last state
        float* srow = a.state + (size_t)a.seq_slot[b] * a.state_stride;
#pragma unroll
        for (int d = 0; d < DMAX; ++d) {
            if (d < D) {
                if (col < V) srow[((size_t)h * D + d) * V + col] = S[d];
                else srow[(size_t)H * D * V + (size_t)h * D + d] = S[d];
            }
        }
    }
}

// every chunk's start state from the run's start state and the chunks' last states
__global__ void __launch_bounds__(128)
memory_chunk_carry_kernel(MemoryChunkArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;        // (row, column)
    if (i >= a.D * a.cols) return;
    const int d = i / a.cols, col = i - d * a.cols;
    const float* srow = a.state + (size_t)a.seq_slot[b] * a.state_stride;
    float S = col < a.V ? srow[((size_t)h * a.D + d) * a.V + col] : srow[(size_t)a.H * a.D * a.V + (size_t)h * a.D + d];
    const int chunks = (a.seq_qlen[b] + a.chunk_len - 1) / a.chunk_len;
    // eight chunks' last states and decays are asked for at once, so that a chunk costs no trip to memory of its own
    for (int k0 = 0; k0 < chunks; k0 += 8) {
        float last[8], decay[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const size_t at = ((size_t)b * a.n_chunks + min(k0 + j, chunks - 1)) * a.H + h;
            last[j] = a.chunk_state[(at * a.D + d) * a.cols + col];
            decay[j] = a.chunk_decay[at * a.D + d];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (k0 + j < chunks) {
                const size_t at = ((size_t)b * a.n_chunks + k0 + j) * a.H + h;
                a.chunk_state[(at * a.D + d) * a.cols + col] = S;
                S = fmaf(decay[j], S, last[j]);
            }
        }
    }
}

// the gated kind's outputs divided by max(|n.q|, e^-m) + 1e-6, all tokens at once
__global__ void __launch_bounds__(256)
memory_divide_kernel(MemoryChunkArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long n = (long long)a.T * a.H * a.V;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long th = i / a.V;
        a.out[i] = a.out[i] / (fmaxf(fabsf(a.nq[th]), a.gates[th * 4 + 2]) + 1e-6f);
    }
}

template <typename TA, int DMAX, int KIND, int NT>
static int launch_memory_chunks_nt(const MemoryChunkArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)MC_TOKENS * (3 * a.D + NT + 2) * sizeof(float);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    const dim3 walk((a.cols + NT - 1) / NT, a.H, a.B * a.n_chunks);
    int rc;
    if (KIND == 0 || KIND == 3) {
        const long long n = (long long)a.T * a.H;
        if (KIND == 0) rc = gl_launch(memory_log_gates_kernel<TA>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, a);
        else rc = gl_launch(memory_decay_gates_kernel<TA>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, a);
        if (rc != 0) return rc;
    }
    if (KIND == 0) {
        rc = gl_launch(memory_gate_walk_kernel, dim3(a.B * a.H), dim3(32), 0, stream, 1, a);
        if (rc != 0) return rc;
    }
    rc = gl_launch(memory_chunk_decay_kernel<TA, KIND>, dim3((a.D + 127) / 128, a.H, a.B * a.n_chunks), dim3(128), 0, stream, 1, a);
    if (rc != 0) return rc;
    const bool full = a.D == DMAX;
    rc = full ? gl_launch_in_order(memory_chunk_walk_kernel<TA, DMAX, KIND, 1, NT, true>, walk, dim3(NT), smem, stream, a)
              : gl_launch_in_order(memory_chunk_walk_kernel<TA, DMAX, KIND, 1, NT, false>, walk, dim3(NT), smem, stream, a);
    if (rc != 0) return rc;
    rc = gl_launch(memory_chunk_carry_kernel, dim3((a.D * a.cols + 127) / 128, a.H, a.B), dim3(128), 0, stream, 1, a);
    if (rc != 0) return rc;
    rc = full ? gl_launch_in_order(memory_chunk_walk_kernel<TA, DMAX, KIND, 2, NT, true>, walk, dim3(NT), smem, stream, a)
              : gl_launch_in_order(memory_chunk_walk_kernel<TA, DMAX, KIND, 2, NT, false>, walk, dim3(NT), smem, stream, a);
    if (rc != 0 || KIND != 0) return rc;
    const long long n = (long long)a.T * a.H * a.V;
    const long long want = (n + 255) / 256;
    return gl_launch(memory_divide_kernel, dim3((unsigned)(want > 16384 ? 16384 : want)), dim3(256), 0, stream, 1, a);
}

template <typename TA, int DMAX, int KIND>
static int launch_memory_chunks(const MemoryChunkArgs& a, cudaStream_t stream) {
    // heads of up to 64 columns (a state-space layer's) would leave half of a block's threads without a column
    if constexpr (KIND == 3) {
        if (a.cols <= 64) return launch_memory_chunks_nt<TA, DMAX, KIND, 64>(a, stream);
    }
    return launch_memory_chunks_nt<TA, DMAX, KIND, MC_THREADS>(a, stream);
}

template <typename TA, int KIND>
static int dispatch_memory_chunks(const MemoryChunkArgs& a, cudaStream_t stream) {
    if (a.D <= 16) return launch_memory_chunks<TA, 16, KIND>(a, stream);
    if (a.D <= 32) return launch_memory_chunks<TA, 32, KIND>(a, stream);
    if (a.D <= 64) return launch_memory_chunks<TA, 64, KIND>(a, stream);
    if (a.D <= 128) return launch_memory_chunks<TA, 128, KIND>(a, stream);
    return GL_ERR_SHAPE;
}

template <typename TA>
static int dispatch_memory_chunks_kind(const MemoryChunkArgs& a, cudaStream_t stream) {
    if (a.kind == 0) return dispatch_memory_chunks<TA, 0>(a, stream);
    if (a.kind == 1) return dispatch_memory_chunks<TA, 1>(a, stream);
    return dispatch_memory_chunks<TA, 3>(a, stream);
}

// (launches 4 kernels for the bounded-forget kind, 5 for the plain decay, 7 for the gated one)
GL_API int gl_memory_chunks(const MemoryChunkArgs* args, int act_dtype, cudaStream_t stream) {
    const MemoryChunkArgs& a = *args;
    if (a.B <= 0 || a.T <= 0) return GL_OK;
    if (a.H <= 0 || a.D <= 0 || a.D > 128 || a.V <= 0 || a.n_chunks <= 0 || a.chunk_len <= 0) return GL_ERR_SHAPE;
    if ((a.kind != 0 && a.kind != 1 && a.kind != 3) || a.cols != a.V + (a.kind == 0 ? 1 : 0)) return GL_ERR_SHAPE;
    if ((long long)a.B * a.n_chunks > 65535 || a.H > 65535) return GL_ERR_SHAPE;
    if (!a.chunk_state || !a.chunk_decay || (a.kind == 0 && (!a.nq || !a.gates || !(a.cap > 0.f)))) return GL_ERR_SHAPE;
    if (a.kind == 3) {
        if (!a.gates || a.KVH <= 0 || a.H % a.KVH) return GL_ERR_SHAPE;
        if ((a.lower != nullptr) == (a.gates_in != nullptr)) return GL_ERR_SHAPE;
        if (a.gates_in && (!a.a_log || !a.dt_bias)) return GL_ERR_SHAPE;
        if (a.cosv && (!a.sinv || a.rot_half <= 0 || 2 * a.rot_half > a.D)) return GL_ERR_SHAPE;
    }
    if (act_dtype == GL_F32) return dispatch_memory_chunks_kind<float>(a, stream);
    if (act_dtype == GL_BF16) return dispatch_memory_chunks_kind<__nv_bfloat16>(a, stream);
    return GL_ERR_DTYPE;
}
