// The gated delta rule with one decay per head and key channel, as a recurrence over a per-request state in float:
//
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          S [dim, vdim] per head
//
// in this order, so the read-out sees the token's own write.  The state is zero before a request's first token and lives
// in the request's state slot between steps, so any cutting of the tokens gives the same recurrence.
//
// The columns of S are independent (column e only meets v_t[e], u[e], o_t[e]), so a column belongs to DG neighbouring
// threads that each keep NR of its rows in registers; the two dot products of a token meet by shuffles.  A block takes
// one span, one head and up to 256 / DG columns, stages 16 tokens of q, k, g, v and beta in shared memory (padded with
// zeros to NR * DG rows, so the inner loop has no bounds) and walks them token by token with 16-byte shared loads.
// Unlike a recurrence with a scalar decay the transition (I - beta k k^T) diag(g) does not commute with anything, so a
// span is walked in order by one block per (head, column block).
//
// Also here: the small second projection of a low-rank pair (x W1^T) W2^T from columns of a fused first projection,
// with what follows it in float: nothing, a sigmoid, or the log decay -rate_h * softplus(z + bias).
#include "common.cuh"
#include "warp_mma.cuh"

namespace {

constexpr int DELTA_STAGE = 16;

// Floats of padding behind the `nr` rows that one of a column's `dg` threads owns in a staged row: it keeps the 16-byte
// reads of the dg threads on different banks (rows of 4 lie side by side without any).
__host__ __device__ constexpr int delta_pad(int nr, int dg) { return (dg > 1 && nr > 4) ? 4 : 0; }

struct DeltaParams {
    const float* q;            // [T, G, dim]
    const float* k;            // [T, G, dim]
    const float* v;            // [T, H, vdim]
    const float* g;            // [T, H, dim] logarithms of the decay factors (<= 0)
    const void* beta;          // row t at beta + t * beta_stride elements: H values before the sigmoid
    long long beta_stride;
    int beta_dtype;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* span_slot;
    float* state;              // a slot's S begins at slot * state_stride + state_off: [H, dim, vdim]
    long long state_stride, state_off;
    float* out;                // [T, H, vdim]
    int H, G, dim, vdim, EV;
    int blocked;               // host: spans are walked in blocks of DELTA_STAGE tokens (delta_rule_blocked_kernel)
    float* scratch;            // blocked: [max_blocks, H, delta_block_floats(dim)] what the first kernel leaves for the second
    int max_blocks;            // blocked: at least sum over the spans of ceil(len / DELTA_STAGE)
    int nr, dg;                // blocked: the second kernel's split of a column (rows a thread, threads a column)
};

template <int NR, int DG>
__global__ void __launch_bounds__(256) delta_rule_kernel(DeltaParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int PADF = delta_pad(NR, DG);
    constexpr int DPAD = DG * (NR + PADF);
    const int span = blockIdx.x, h = blockIdx.y;
    const int dim = p.dim, vdim = p.vdim;
    const int len = p.span_len[span], row0 = p.span_row[span], pos0 = p.span_pos[span];
    float* qs = sm;                              // [STAGE][DPAD]
    float* ks = qs + DELTA_STAGE * DPAD;
    float* gs = ks + DELTA_STAGE * DPAD;
    float* vs = gs + DELTA_STAGE * DPAD;         // [STAGE][EV]
    float* bs = vs + DELTA_STAGE * p.EV;         // [STAGE]
    const int dg = threadIdx.x % DG, el = threadIdx.x / DG;
    const int e = blockIdx.z * p.EV + el;
    const bool live = el < p.EV && e < vdim;
    const int hk = h / (p.H / p.G);
    float* slot = p.state + (long long)p.span_slot[span] * p.state_stride + p.state_off + (size_t)h * dim * vdim;

    float S[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = dg * NR + j;
        S[j] = (pos0 > 0 && live && d < dim) ? slot[(size_t)d * vdim + e] : 0.0f;
    }
    for (int i = threadIdx.x; i < 3 * DELTA_STAGE * DPAD; i += blockDim.x) sm[i] = 0.0f;     // the padding stays zero
    auto at = [](int d) { return (d / NR) * (NR + PADF) + d % NR; };
    for (int c0 = 0; c0 < len; c0 += DELTA_STAGE) {
        const int n = min(DELTA_STAGE, len - c0);
        __syncthreads();
        for (int it = threadIdx.x; it < n * dim; it += blockDim.x) {
            const int tl = it / dim, d = it - tl * dim;
            const size_t row = (size_t)(row0 + c0 + tl);
            qs[tl * DPAD + at(d)] = p.q[(row * p.G + hk) * dim + d];
            ks[tl * DPAD + at(d)] = p.k[(row * p.G + hk) * dim + d];
            gs[tl * DPAD + at(d)] = expf(p.g[(row * p.H + h) * dim + d]);
        }
        for (int it = threadIdx.x; it < n * p.EV; it += blockDim.x) {
            const int tl = it / p.EV, cc = it - tl * p.EV;
            const int ee = blockIdx.z * p.EV + cc;
            vs[it] = ee < vdim ? p.v[((size_t)(row0 + c0 + tl) * p.H + h) * vdim + ee] : 0.0f;
        }
        if (threadIdx.x < n) {
            const size_t at_b = (size_t)(row0 + c0 + threadIdx.x) * p.beta_stride + h;
            const float z = p.beta_dtype == LLB_F32 ? ((const float*)p.beta)[at_b]
                                                    : __bfloat162float(((const __nv_bfloat16*)p.beta)[at_b]);
            bs[threadIdx.x] = 1.0f / (1.0f + expf(-z));
        }
        __syncthreads();
        for (int tl = 0; tl < n; ++tl) {
            const float vv = el < p.EV ? vs[tl * p.EV + el] : 0.0f;
            const float beta = bs[tl];
            const float4* k4p = reinterpret_cast<const float4*>(ks + tl * DPAD + dg * (NR + PADF));
            const float4* q4p = reinterpret_cast<const float4*>(qs + tl * DPAD + dg * (NR + PADF));
            const float4* g4p = reinterpret_cast<const float4*>(gs + tl * DPAD + dg * (NR + PADF));
            float4 kk[NR / 4];
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int j = 0; j < NR; j += 4) {
                const float4 g4 = g4p[j >> 2];
                const float4 k4 = kk[j >> 2] = k4p[j >> 2];
                S[j] *= g4.x; S[j + 1] *= g4.y; S[j + 2] *= g4.z; S[j + 3] *= g4.w;
                a0 = fmaf(S[j], k4.x, a0); a1 = fmaf(S[j + 1], k4.y, a1);
                a2 = fmaf(S[j + 2], k4.z, a2); a3 = fmaf(S[j + 3], k4.w, a3);
            }
            float dot = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int o = DG >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float u = beta * (vv - dot);
            a0 = a1 = a2 = a3 = 0.0f;
#pragma unroll
            for (int j = 0; j < NR; j += 4) {
                const float4 k4 = kk[j >> 2];
                const float4 q4 = q4p[j >> 2];
                S[j] = fmaf(k4.x, u, S[j]); S[j + 1] = fmaf(k4.y, u, S[j + 1]);
                S[j + 2] = fmaf(k4.z, u, S[j + 2]); S[j + 3] = fmaf(k4.w, u, S[j + 3]);
                a0 = fmaf(S[j], q4.x, a0); a1 = fmaf(S[j + 1], q4.y, a1);
                a2 = fmaf(S[j + 2], q4.z, a2); a3 = fmaf(S[j + 3], q4.w, a3);
            }
            float o = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int s = DG >> 1; s > 0; s >>= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
            if (live && dg == 0) p.out[((size_t)(row0 + c0 + tl) * p.H + h) * vdim + e] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int d = dg * NR + j;
            if (d < dim) slot[(size_t)d * vdim + e] = S[j];
        }
    }
}

// The same recurrence over blocks of DELTA_STAGE tokens at a time, for spans long enough that walking them token by token
// leaves the GPU waiting on one dependent chain per token.  With L_t the running sum of the log decays inside a block
// (L_0 = 0) and S_0 the state before it, unrolling the recurrence gives
//
//     u_t = beta_t (v_t - S_0^T (e^{L_t} k_t) - sum_{s<t} A_ts u_s)        A_ts = sum_d k_t[d] k_s[d] e^{L_t[d] - L_s[d]}
//     o_t = S_0^T (e^{L_t} q_t) + sum_{s<=t} M_ts u_s                       M_ts = sum_d q_t[d] k_s[d] e^{L_t[d] - L_s[d]}
//     S_n = diag(e^{L_n}) S_0 + sum_s (e^{L_n - L_s} k_s) u_s^T
//
// A, M and the scaled rows belong to the head and the block of tokens, not to the state: a first kernel makes them for
// all blocks of all spans side by side (every exponent is <= 0, so nothing overflows however fast a channel decays) and
// leaves them in scratch; the second kernel walks a span's blocks in order, and for each block every column runs three
// passes whose terms are independent across the block's tokens (the products with S_0, the read-out, the new state)
// around one short forward substitution for u.  Block b of the step is block c of span s when the spans before s hold
// b - c blocks: both kernels count the same way, so no list of blocks is needed from the host.
constexpr int DELTA_PAIRS = DELTA_STAGE * (DELTA_STAGE + 1) / 2;

// Floats that the first kernel leaves per (block of tokens, head), already in the second kernel's shared-memory layout:
// three matrices [C][dpad] (a row's `dim` numbers in dg groups of nr, each padded by 4), one row [dpad], then A and M.
__host__ __device__ inline long long delta_block_floats(int dpad) {
    return 3ll * DELTA_STAGE * dpad + dpad + 2 * DELTA_STAGE * DELTA_STAGE;
}

__global__ void __launch_bounds__(256) delta_blocks_prepare_kernel(DeltaParams p, int num_spans) {
    extern __shared__ __align__(16) float sm[];
    constexpr int C = DELTA_STAGE;
    const int dim = p.dim, h = blockIdx.y;
    const int RS = dim + 1;                      // row pitch: the rows of a warp's pairs on different banks
    int span = 0, c = blockIdx.x;
    while (span < num_spans) {
        const int blocks = (p.span_len[span] + C - 1) / C;
        if (c < blocks) break;
        c -= blocks;
        ++span;
    }
    if (span >= num_spans) return;
    const int len = p.span_len[span], row0 = p.span_row[span] + c * C;
    const int n = min(C, len - c * C);
    const int hk = h / (p.H / p.G);
    float* kr = sm;                              // [C][RS]    k_t
    float* qr = kr + C * RS;                     // [C][RS]    q_t
    float* Ls = qr + C * RS;                     // [C][RS]    log decays, then their running sums L_t
    const int nr = p.nr, padded = p.nr + delta_pad(p.nr, p.dg), dpad = p.dg * padded;
    float* dst = p.scratch + ((size_t)blockIdx.x * p.H + h) * delta_block_floats(dpad);
    float* Qb = dst;                             // [C][dpad]  e^{L_t} q_t
    float* Kb = Qb + C * dpad;                   // [C][dpad]  e^{L_t} k_t
    float* Kp = Kb + C * dpad;                   // [C][dpad]  e^{L_n - L_t} k_t
    float* GC = Kp + C * dpad;                   // [dpad]     e^{L_n}
    float* As = GC + dpad;                       // [C][C]     A_ts at [s][t] (s < t), else 0: a row holds what u_s adds to
    float* Ms = As + C * C;                      // [C][C]     M_ts at [s][t] (s <= t), else 0    the tokens after it
    for (int it = threadIdx.x; it < C * dim; it += blockDim.x) {
        const int tl = it / dim, d = it - tl * dim;
        const size_t row = (size_t)(row0 + tl);
        const bool in = tl < n;
        kr[tl * RS + d] = in ? p.k[(row * p.G + hk) * dim + d] : 0.0f;
        qr[tl * RS + d] = in ? p.q[(row * p.G + hk) * dim + d] : 0.0f;
        Ls[tl * RS + d] = in ? p.g[(row * p.H + h) * dim + d] : 0.0f;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {          // running sums of the log decays
        float run = 0.0f;
        for (int tl = 0; tl < C; ++tl) {
            run += Ls[tl * RS + d];
            Ls[tl * RS + d] = run;
        }
    }
    __syncthreads();
    for (int it = threadIdx.x; it < C * dim; it += blockDim.x) {
        const int tl = it / dim, d = it - tl * dim;
        const float L = Ls[tl * RS + d], Ln = Ls[(C - 1) * RS + d];          // rows past n add nothing: L stays L_n
        const float eL = expf(L);
        const int col = (d / nr) * padded + d % nr;
        Kb[tl * dpad + col] = eL * kr[tl * RS + d];
        Qb[tl * dpad + col] = eL * qr[tl * RS + d];
        Kp[tl * dpad + col] = expf(Ln - L) * kr[tl * RS + d];
        if (tl == 0) GC[col] = expf(Ln);
    }
    for (int it = threadIdx.x; it < (C + 1) * dpad; it += blockDim.x) {          // the padding is zero
        const int col = it % dpad, tl = it / dpad;
        if (col % padded >= nr || (col / padded) * nr + col % padded >= dim) {
            if (tl < C) Qb[it] = Kb[it] = Kp[it] = 0.0f;
            else GC[col] = 0.0f;
        }
    }
    for (int pr = threadIdx.x; pr < C * C; pr += blockDim.x) {
        const int s = pr / C, t = pr - s * C;
        if (s > t) As[pr] = Ms[pr] = 0.0f;
    }
    for (int pr = threadIdx.x; pr < DELTA_PAIRS; pr += blockDim.x) {          // the pairs s <= t, packed: no idle lanes
        int t = (int)((sqrtf(8.0f * pr + 1.0f) - 1.0f) * 0.5f);
        while (t * (t + 1) / 2 > pr) --t;
        while ((t + 1) * (t + 2) / 2 <= pr) ++t;
        const int s = pr - t * (t + 1) / 2;
        float a = 0.0f, m = 0.0f;
        if (t < n) {
            for (int d = 0; d < dim; ++d) {
                const float w = kr[s * RS + d] * expf(Ls[t * RS + d] - Ls[s * RS + d]);
                a = fmaf(kr[t * RS + d], w, a);
                m = fmaf(qr[t * RS + d], w, m);
            }
        }
        As[s * C + t] = s < t ? a : 0.0f;
        Ms[s * C + t] = m;
    }
}

template <int NR, int DG>
__global__ void __launch_bounds__(64) delta_rule_blocked_kernel(DeltaParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int C = DELTA_STAGE;
    constexpr int PADF = delta_pad(NR, DG);
    constexpr int DPAD = DG * (NR + PADF);
    const int span = blockIdx.x, h = blockIdx.y;
    const int dim = p.dim, vdim = p.vdim;
    const int len = p.span_len[span], row0 = p.span_row[span], pos0 = p.span_pos[span];
    int first_block = 0;                         // of this span among the step's blocks (as the first kernel counts them)
    for (int s = 0; s < span; ++s) first_block += (p.span_len[s] + C - 1) / C;
    constexpr int BLOCK_FLOATS = 3 * C * DPAD + DPAD + 2 * C * C;          // = delta_block_floats(DPAD): one copy of 16-byte pieces
    const int stage_floats = BLOCK_FLOATS + C * p.EV + C;                  // + v [C][EV] and beta [C]
    const int stage_pitch = (stage_floats + 3) & ~3;
    const int dg = threadIdx.x % DG, el = threadIdx.x / DG;
    const int e = blockIdx.z * p.EV + el;
    const bool live = el < p.EV && e < vdim;
    float* slot = p.state + (long long)p.span_slot[span] * p.state_stride + p.state_off + (size_t)h * dim * vdim;

    float S[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = dg * NR + j;
        S[j] = (pos0 > 0 && live && d < dim) ? slot[(size_t)d * vdim + e] : 0.0f;
    }
    // Two stages in shared memory: while a block of tokens is worked on, the next one's matrices arrive by cp.async and its
    // values and betas wait in registers.
    auto fetch = [&](int blk, int stage) {
        const float* src = p.scratch + ((size_t)blk * p.H + h) * BLOCK_FLOATS;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(sm + stage * stage_pitch);
        for (int i = threadIdx.x; i < BLOCK_FLOATS / 4; i += blockDim.x) wm::cp_async16(dst + i * 16, src + i * 4, true);
        wm::cp_async_commit();
    };
    constexpr int VPT = (C * 64 / DG + 63) / 64;                           // values a thread carries for the next block
    float vnext[VPT], bnext = 0.0f;
    auto load_vb = [&](int c0) {
        const int n = min(C, len - c0);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int it = threadIdx.x + i * blockDim.x;
            const int tl = it / p.EV, cc = it - tl * p.EV;
            const int ee = blockIdx.z * p.EV + cc;
            vnext[i] = (it < C * p.EV && tl < n && ee < vdim) ? p.v[((size_t)(row0 + c0 + tl) * p.H + h) * vdim + ee] : 0.0f;
        }
        bnext = -INFINITY;          // (its sigmoid is 0; taken when the value is stored, not while the load is in flight)
        if (threadIdx.x < n) {
            const size_t at_b = (size_t)(row0 + c0 + threadIdx.x) * p.beta_stride + h;
            bnext = p.beta_dtype == LLB_F32 ? ((const float*)p.beta)[at_b] : __bfloat162float(((const __nv_bfloat16*)p.beta)[at_b]);
        }
    };
    auto store_vb = [&](int stage) {
        float* vsn = sm + stage * stage_pitch + BLOCK_FLOATS;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int it = threadIdx.x + i * blockDim.x;
            if (it < C * p.EV) vsn[it] = vnext[i];
        }
        if (threadIdx.x < C) vsn[C * p.EV + threadIdx.x] = 1.0f / (1.0f + expf(-bnext));
    };
    fetch(first_block, 0);
    load_vb(0);
    store_vb(0);
    for (int c0 = 0, blk = first_block, stage = 0; c0 < len; c0 += C, ++blk, stage ^= 1) {
        const int n = min(C, len - c0);
        const bool more = c0 + C < len;
        if (more) {
            fetch(blk + 1, stage ^ 1);          // (the stage it lands in was last read before the barrier that ended the block before)
            load_vb(c0 + C);
            wm::cp_async_wait<1>();
        } else {
            wm::cp_async_wait<0>();
        }
        __syncthreads();
        const float* Qb = sm + stage * stage_pitch;          // [C][DPAD]
        const float* Kb = Qb + C * DPAD;                       // [C][DPAD]
        const float* Kp = Kb + C * DPAD;                       // [C][DPAD]
        const float* GC = Kp + C * DPAD;                       // [DPAD]
        const float* As = GC + DPAD;                           // [C][C]
        const float* Ms = As + C * C;                          // [C][C]
        const float* vs = Ms + C * C;                          // [C][EV]
        const float* bs = vs + C * p.EV;                       // [C]
        // what the state before the block gives every token: w_t = v_t - S_0^T (e^{L_t} k_t), o_t = S_0^T (e^{L_t} q_t)
        float w[C], o[C];
#pragma unroll
        for (int t = 0; t < C; ++t) {
            const float4* k4p = reinterpret_cast<const float4*>(Kb + t * DPAD + dg * (NR + PADF));
            const float4* q4p = reinterpret_cast<const float4*>(Qb + t * DPAD + dg * (NR + PADF));
            float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
            for (int j = 0; j < NR; j += 4) {
                const float4 k4 = k4p[j >> 2], q4 = q4p[j >> 2];
                a0 = fmaf(S[j], k4.x, a0); a1 = fmaf(S[j + 1], k4.y, a1);
                a0 = fmaf(S[j + 2], k4.z, a0); a1 = fmaf(S[j + 3], k4.w, a1);
                b0 = fmaf(S[j], q4.x, b0); b1 = fmaf(S[j + 1], q4.y, b1);
                b0 = fmaf(S[j + 2], q4.z, b0); b1 = fmaf(S[j + 3], q4.w, b1);
            }
            w[t] = a0 + a1;
            o[t] = b0 + b1;
        }
#pragma unroll
        for (int t = 0; t < C; ++t) {
#pragma unroll
            for (int sh = DG >> 1; sh > 0; sh >>= 1) {
                w[t] += __shfl_xor_sync(0xffffffffu, w[t], sh);
                o[t] += __shfl_xor_sync(0xffffffffu, o[t], sh);
            }
            w[t] = (el < p.EV ? vs[t * p.EV + el] : 0.0f) - w[t];
        }
        // forward substitution (every lane of a column computes the same u) and the read-out's part from inside the block,
        // token s at a time: once u_s is known it is taken off every later token's right side and added to every later
        // token's output, which are independent of one another (a token's sums still run over s in rising order)
        float u[C];
#pragma unroll
        for (int s = 0; s < C; ++s) {
            u[s] = bs[s] * w[s];
#pragma unroll
            for (int t4 = (s / 4) * 4; t4 < C; t4 += 4) {
                const float4 a4 = *reinterpret_cast<const float4*>(As + s * C + t4);
                const float4 m4 = *reinterpret_cast<const float4*>(Ms + s * C + t4);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w}, mv[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int t = t4 + i;
                    if (t > s) w[t] = fmaf(-av[i], u[s], w[t]);
                    if (t >= s) o[t] = fmaf(mv[i], u[s], o[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < C; ++t)
            if (live && dg == 0 && t < n) p.out[((size_t)(row0 + c0 + t) * p.H + h) * vdim + e] = o[t];
        // the state after the block
        {
            const float4* g4p = reinterpret_cast<const float4*>(GC + dg * (NR + PADF));
#pragma unroll
            for (int j = 0; j < NR; j += 4) {
                const float4 g4 = g4p[j >> 2];
                S[j] *= g4.x; S[j + 1] *= g4.y; S[j + 2] *= g4.z; S[j + 3] *= g4.w;
            }
#pragma unroll
            for (int t = 0; t < C; ++t) {
                const float4* k4p = reinterpret_cast<const float4*>(Kp + t * DPAD + dg * (NR + PADF));
#pragma unroll
                for (int j = 0; j < NR; j += 4) {
                    const float4 k4 = k4p[j >> 2];
                    S[j] = fmaf(k4.x, u[t], S[j]); S[j + 1] = fmaf(k4.y, u[t], S[j + 1]);
                    S[j + 2] = fmaf(k4.z, u[t], S[j + 2]); S[j + 3] = fmaf(k4.w, u[t], S[j + 3]);
                }
            }
        }
        if (more) store_vb(stage ^ 1);
        __syncthreads();          // every thread has read this stage: the block after next may land in it
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int d = dg * NR + j;
            if (d < dim) slot[(size_t)d * vdim + e] = S[j];
        }
    }
}

template <int NR, int DG>
int launch_delta(const DeltaParams& p0, int num_spans, cudaStream_t stream) {
    DeltaParams p = p0;
    const int cols = 256 / DG;
    p.EV = p.vdim < cols ? p.vdim : cols;
    constexpr int PADF = delta_pad(NR, DG);
    const size_t smem = (size_t)(3 * DELTA_STAGE * DG * (NR + PADF) + DELTA_STAGE * p.EV + DELTA_STAGE) * sizeof(float);
    const int threads = ((p.EV * DG + 31) / 32) * 32;
    const dim3 grid(num_spans, p.H, (p.vdim + p.EV - 1) / p.EV);
    if (p.blocked) {
        // two warps a block: what paces a block is its own chain of blocks of tokens, so the columns are spread over as
        // many multiprocessors as there are; the first kernel has made what all of a head's columns share
        constexpr int C = DELTA_STAGE;
        const int cols_b = 64 / DG;
        p.EV = p.vdim < cols_b ? p.vdim : cols_b;
        const int threads_b = ((p.EV * DG + 31) / 32) * 32;
        const dim3 grid_b(num_spans, p.H, (p.vdim + p.EV - 1) / p.EV);
        const size_t pre_bytes = (size_t)3 * C * (p.dim + 1) * sizeof(float);
        if (pre_bytes > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(delta_blocks_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       (int)pre_bytes);
            if (e != cudaSuccess) return llb_fail("delta_rule: %s", cudaGetErrorString(e));
        }
        p.nr = NR; p.dg = DG;
        delta_blocks_prepare_kernel<<<dim3(p.max_blocks, p.H), 256, pre_bytes, stream>>>(p, num_spans);
        int rc = llb_check_launch("delta_blocks_prepare");
        if (rc) return rc;
        const size_t stage = ((size_t)delta_block_floats(DG * (NR + PADF)) + C * p.EV + C + 3) & ~(size_t)3;
        const size_t bytes = 2 * stage * sizeof(float);
        if (bytes > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(delta_rule_blocked_kernel<NR, DG>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return llb_fail("delta_rule: %s", cudaGetErrorString(e));
        }
        delta_rule_blocked_kernel<NR, DG><<<grid_b, threads_b, bytes, stream>>>(p);
        return llb_check_launch("delta_rule_blocked");
    }
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<NR, DG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return llb_fail("delta_rule: %s", cudaGetErrorString(e));
    }
    delta_rule_kernel<NR, DG><<<grid, threads, smem, stream>>>(p);
    return llb_check_launch("delta_rule");
}

struct LowRankParams {
    const void* x;             // row t at x + t * x_stride elements; R inputs from column x_off on
    long long x_stride;
    int x_off, R, N, per_rate;
    const void* w;             // [N, R]
    const float* bias;         // [N] or null
    const float* rate;         // [N / per_rate] (mode 2)
    void* out;                 // [T, N]
    int mode;
};

// A block takes LR_ROWS rows of x (their R inputs in shared memory, padded to a multiple of 4) and 256 outputs; a thread
// owns one output for all the block's rows, so a weight is loaded once for LR_ROWS products and the inputs come as
// 16-byte broadcast reads.
constexpr int LR_ROWS = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) low_rank_up_kernel(LowRankParams p, int T) {
    extern __shared__ __align__(16) float xs[];      // [LR_ROWS][R4]
    const int R4 = (p.R + 3) & ~3;
    const int t0 = blockIdx.y * LR_ROWS;
    const int rows = min(LR_ROWS, T - t0);
    for (int i = threadIdx.x; i < LR_ROWS * R4; i += blockDim.x) {
        const int tl = i / R4, r = i - tl * R4;
        xs[i] = (tl < rows && r < p.R) ? llb_to_float(((const TX*)p.x)[(size_t)(t0 + tl) * p.x_stride + p.x_off + r]) : 0.0f;
    }
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= p.N) return;
    const TW* wr = (const TW*)p.w + (size_t)n * p.R;
    float acc[LR_ROWS];
#pragma unroll
    for (int tl = 0; tl < LR_ROWS; ++tl) acc[tl] = 0.0f;
#pragma unroll 4
    for (int r = 0; r < R4; r += 4) {          // (unrolled: the weights of four steps are asked for before the first is used)
        float w4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w4[j] = r + j < p.R ? llb_to_float(wr[r + j]) : 0.0f;
#pragma unroll
        for (int tl = 0; tl < LR_ROWS; ++tl) {
            const float4 x4 = *reinterpret_cast<const float4*>(xs + tl * R4 + r);
            acc[tl] = fmaf(x4.x, w4[0], acc[tl]);
            acc[tl] = fmaf(x4.y, w4[1], acc[tl]);
            acc[tl] = fmaf(x4.z, w4[2], acc[tl]);
            acc[tl] = fmaf(x4.w, w4[3], acc[tl]);
        }
    }
    const float bias = p.bias ? p.bias[n] : 0.0f;
    const float rate = p.mode == 2 ? p.rate[n / p.per_rate] : 0.0f;
#pragma unroll
    for (int tl = 0; tl < LR_ROWS; ++tl) {
        if (tl >= rows) break;
        float z = acc[tl] + bias;
        if (p.mode == 1) {
            z = 1.0f / (1.0f + expf(-z));
        } else if (p.mode == 2) {
            const float sp = z > 20.0f ? z : log1pf(expf(z));
            z = -rate * sp;
        }
        ((TO*)p.out)[(size_t)(t0 + tl) * p.N + n] = llb_from_float<TO>(z);
    }
}

__device__ __forceinline__ float low_rank_finish(const LowRankParams& p, int n, float z) {
    if (p.bias) z += p.bias[n];
    if (p.mode == 1) return 1.0f / (1.0f + expf(-z));
    if (p.mode == 2) return -p.rate[n / p.per_rate] * (z > 20.0f ? z : log1pf(expf(z)));
    return z;
}

// Few rows (a decode step): a warp an output, the lanes along the R inputs, so that a weight row is one coalesced read
// and a step's few thousand outputs are spread over a hundred blocks instead of four.
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) low_rank_up_few_rows_kernel(LowRankParams p, int T) {
    extern __shared__ __align__(16) float xs[];      // [T][R]
    for (int i = threadIdx.x; i < T * p.R; i += blockDim.x) {
        const int tl = i / p.R, r = i - tl * p.R;
        xs[i] = llb_to_float(((const TX*)p.x)[(size_t)tl * p.x_stride + p.x_off + r]);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= p.N) return;
    const TW* wr = (const TW*)p.w + (size_t)n * p.R;
    float wv[16];                                    // R <= 512: at most 16 inputs a lane
#pragma unroll
    for (int i = 0; i < 16; ++i) wv[i] = lane + 32 * i < p.R ? llb_to_float(wr[lane + 32 * i]) : 0.0f;
    for (int tl = 0; tl < T; ++tl) {
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (lane + 32 * i < p.R) acc = fmaf(xs[tl * p.R + lane + 32 * i], wv[i], acc);
        acc = llb_warp_sum(acc);
        if (lane == 0) ((TO*)p.out)[(size_t)tl * p.N + n] = llb_from_float<TO>(low_rank_finish(p, n, acc));
    }
}

template <typename TX, typename TW>
int launch_low_rank(const LowRankParams& p, int T, int out_dtype, cudaStream_t stream) {
    if (T <= LR_ROWS) {
        const dim3 grid_f((p.N + 7) / 8);
        const size_t smem_f = (size_t)T * p.R * sizeof(float);
        if (out_dtype == LLB_F32) low_rank_up_few_rows_kernel<TX, TW, float><<<grid_f, 256, smem_f, stream>>>(p, T);
        else low_rank_up_few_rows_kernel<TX, TW, __nv_bfloat16><<<grid_f, 256, smem_f, stream>>>(p, T);
        return llb_check_launch("low_rank_up_few_rows");
    }
    const dim3 grid((p.N + 255) / 256, (T + LR_ROWS - 1) / LR_ROWS);
    const size_t smem = (size_t)LR_ROWS * ((p.R + 3) & ~3) * sizeof(float);
    if (out_dtype == LLB_F32) low_rank_up_kernel<TX, TW, float><<<grid, 256, smem, stream>>>(p, T);
    else low_rank_up_kernel<TX, TW, __nv_bfloat16><<<grid, 256, smem, stream>>>(p, T);
    return llb_check_launch("low_rank_up");
}

}  // namespace

// q, k float [T, G, dim]; v float [T, H, vdim]; g float [T, H, dim] (the logarithms of the decay factors, <= 0); blocked != 0
// walks the spans in blocks of tokens (for steps with long spans; the result is the same recurrence) and needs scratch of
// llb_delta_rule_scratch_floats(max_blocks, H, dim) floats, max_blocks >= sum over spans of ceil(len / 16) (T / 16 +
// num_spans always suffices); beta: the H values
// before the sigmoid of row t at beta + t * beta_stride (float or bf16); the spans of the step; state: float base of the
// state plane, state_stride floats a slot, a slot's S [H, dim, vdim] at state_off; out float [T, H, vdim].
LLB_EXPORT int llb_delta_rule(const float* q, const float* k, const float* v, const float* g, const void* beta,
                              long long beta_stride, int beta_dtype, const int* span_row, const int* span_len,
                              const int* span_pos, const int* span_slot, int num_spans, int H, int G, int dim, int vdim,
                              float* state, long long state_stride, long long state_off, float* out, int blocked,
                              float* scratch, int max_blocks, cudaStream_t stream) {
    if (num_spans == 0) return 0;
    LLB_REQUIRE(q && k && v && g && beta && state && out && span_row && span_len && span_pos && span_slot,
                "delta_rule: bad arguments");
    LLB_REQUIRE(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0, "delta_rule: bad sizes H=%d G=%d dim=%d vdim=%d", H, G, dim, vdim);
    LLB_REQUIRE(dim <= 256, "delta_rule: heads of %d key channels; at most 256", dim);
    LLB_REQUIRE(beta_dtype == LLB_F32 || beta_dtype == LLB_BF16, "delta_rule: unknown dtype %d", beta_dtype);
    DeltaParams p;
    p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta; p.beta_stride = beta_stride; p.beta_dtype = beta_dtype;
    p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.state = state; p.state_stride = state_stride; p.state_off = state_off; p.out = out;
    p.H = H; p.G = G; p.dim = dim; p.vdim = vdim; p.EV = 0; p.blocked = blocked;
    p.scratch = scratch; p.max_blocks = max_blocks;
    LLB_REQUIRE(!blocked || (scratch && max_blocks > 0), "delta_rule: the blocked walk needs scratch");
    if (blocked) {          // more threads a column: what paces a block of tokens is a warp's own instruction chain
        if (dim <= 16) return launch_delta<4, 4>(p, num_spans, stream);
        if (dim <= 32) return launch_delta<4, 8>(p, num_spans, stream);
        if (dim <= 64) return launch_delta<4, 16>(p, num_spans, stream);
        if (dim <= 128) return launch_delta<8, 16>(p, num_spans, stream);
        return launch_delta<16, 16>(p, num_spans, stream);
    }
    if (dim <= 16) return launch_delta<16, 1>(p, num_spans, stream);
    if (dim <= 32) return launch_delta<16, 2>(p, num_spans, stream);
    if (dim <= 64) return launch_delta<16, 4>(p, num_spans, stream);
    if (dim <= 128) return launch_delta<16, 8>(p, num_spans, stream);
    return launch_delta<32, 8>(p, num_spans, stream);
}

LLB_EXPORT long long llb_delta_rule_scratch_floats(int max_blocks, int H, int dim) {
    const int nr = dim <= 64 ? 4 : dim <= 128 ? 8 : 16;          // as llb_delta_rule picks them
    const int dg = dim <= 16 ? 4 : dim <= 32 ? 8 : 16;
    return (long long)max_blocks * H * delta_block_floats(dg * (nr + delta_pad(nr, dg)));
}

// out[t, n] = f(sum_r x[t, x_off + r] * w[n, r] + bias[n]) for T rows of x (row stride x_stride elements, float or bf16),
// w [N, R] float or bf16, bias float [N] or null, out [T, N] float or bf16.  mode 0: f = identity; 1: sigmoid;
// 2: -rate[n / per_rate] * softplus(.), the logarithm of a decay factor, rate float [N / per_rate].
LLB_EXPORT int llb_low_rank_up(const void* x, int x_dtype, long long x_stride, int x_off, int T, int R, const void* w,
                               int w_dtype, int N, const float* bias, int mode, const float* rate, int per_rate,
                               void* out, int out_dtype, cudaStream_t stream) {
    if (T == 0 || N == 0) return 0;
    LLB_REQUIRE(T > 0 && R > 0 && N > 0 && x && w && out, "low_rank_up: bad arguments");
    LLB_REQUIRE(mode >= 0 && mode <= 2 && (mode != 2 || (rate && per_rate > 0)), "low_rank_up: bad mode %d", mode);
    LLB_REQUIRE(R <= 512, "low_rank_up: %d inputs; at most 512 (the first half of a low-rank pair is narrow)", R);
    LLB_REQUIRE(out_dtype == LLB_F32 || out_dtype == LLB_BF16, "low_rank_up: unknown output dtype %d", out_dtype);
    LowRankParams p;
    p.x = x; p.x_stride = x_stride; p.x_off = x_off; p.R = R; p.N = N; p.per_rate = per_rate; p.w = w; p.bias = bias;
    p.rate = rate; p.out = out; p.mode = mode;
    if (x_dtype == LLB_F32 && w_dtype == LLB_F32) return launch_low_rank<float, float>(p, T, out_dtype, stream);
    if (x_dtype == LLB_BF16 && w_dtype == LLB_BF16) return launch_low_rank<__nv_bfloat16, __nv_bfloat16>(p, T, out_dtype, stream);
    if (x_dtype == LLB_BF16 && w_dtype == LLB_F32) return launch_low_rank<__nv_bfloat16, float>(p, T, out_dtype, stream);
    if (x_dtype == LLB_F32 && w_dtype == LLB_BF16) return launch_low_rank<float, __nv_bfloat16>(p, T, out_dtype, stream);
    return llb_fail("low_rank_up: unknown dtypes %d, %d", x_dtype, w_dtype);
}
