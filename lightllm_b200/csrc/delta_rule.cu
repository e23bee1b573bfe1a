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
// with what follows it in float: nothing, a sigmoid, or the decay exp(-rate_h * softplus(z + bias)).
#include "common.cuh"

namespace {

constexpr int DELTA_STAGE = 16;

struct DeltaParams {
    const float* q;            // [T, G, dim]
    const float* k;            // [T, G, dim]
    const float* v;            // [T, H, vdim]
    const float* g;            // [T, H, dim] decay factors
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
};

template <int NR, int DG>
__global__ void __launch_bounds__(256) delta_rule_kernel(DeltaParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int PADF = DG > 1 ? 4 : 0;                 // keeps the DG threads of a column on different banks
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
            gs[tl * DPAD + at(d)] = p.g[(row * p.H + h) * dim + d];
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

template <int NR, int DG>
int launch_delta(const DeltaParams& p0, int num_spans, cudaStream_t stream) {
    DeltaParams p = p0;
    const int cols = 256 / DG;
    p.EV = p.vdim < cols ? p.vdim : cols;
    constexpr int PADF = DG > 1 ? 4 : 0;
    const size_t smem = (size_t)(3 * DELTA_STAGE * DG * (NR + PADF) + DELTA_STAGE * p.EV + DELTA_STAGE) * sizeof(float);
    const int threads = ((p.EV * DG + 31) / 32) * 32;
    const dim3 grid(num_spans, p.H, (p.vdim + p.EV - 1) / p.EV);
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

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) low_rank_up_kernel(LowRankParams p) {
    extern __shared__ float xs[];                    // [R]
    const int t = blockIdx.y;
    const TX* xr = (const TX*)p.x + (size_t)t * p.x_stride + p.x_off;
    for (int r = threadIdx.x; r < p.R; r += blockDim.x) xs[r] = llb_to_float(xr[r]);
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= p.N) return;
    const TW* wr = (const TW*)p.w + (size_t)n * p.R;
    float a0 = 0.0f, a1 = 0.0f;
    int r = 0;
    for (; r + 1 < p.R; r += 2) {
        a0 = fmaf(xs[r], llb_to_float(wr[r]), a0);
        a1 = fmaf(xs[r + 1], llb_to_float(wr[r + 1]), a1);
    }
    if (r < p.R) a0 = fmaf(xs[r], llb_to_float(wr[r]), a0);
    float z = a0 + a1;
    if (p.bias) z += p.bias[n];
    if (p.mode == 1) {
        z = 1.0f / (1.0f + expf(-z));
    } else if (p.mode == 2) {
        const float sp = z > 20.0f ? z : log1pf(expf(z));
        z = expf(-p.rate[n / p.per_rate] * sp);
    }
    ((TO*)p.out)[(size_t)t * p.N + n] = llb_from_float<TO>(z);
}

template <typename TX, typename TW>
int launch_low_rank(const LowRankParams& p, int T, int out_dtype, cudaStream_t stream) {
    const dim3 grid((p.N + 255) / 256, T);
    const size_t smem = (size_t)p.R * sizeof(float);
    if (out_dtype == LLB_F32) low_rank_up_kernel<TX, TW, float><<<grid, 256, smem, stream>>>(p);
    else low_rank_up_kernel<TX, TW, __nv_bfloat16><<<grid, 256, smem, stream>>>(p);
    return llb_check_launch("low_rank_up");
}

}  // namespace

// q, k float [T, G, dim]; v float [T, H, vdim]; g float [T, H, dim] (the decay factors themselves); beta: the H values
// before the sigmoid of row t at beta + t * beta_stride (float or bf16); the spans of the step; state: float base of the
// state plane, state_stride floats a slot, a slot's S [H, dim, vdim] at state_off; out float [T, H, vdim].
LLB_EXPORT int llb_delta_rule(const float* q, const float* k, const float* v, const float* g, const void* beta,
                              long long beta_stride, int beta_dtype, const int* span_row, const int* span_len,
                              const int* span_pos, const int* span_slot, int num_spans, int H, int G, int dim, int vdim,
                              float* state, long long state_stride, long long state_off, float* out,
                              cudaStream_t stream) {
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
    p.H = H; p.G = G; p.dim = dim; p.vdim = vdim; p.EV = 0;
    if (dim <= 16) return launch_delta<16, 1>(p, num_spans, stream);
    if (dim <= 32) return launch_delta<16, 2>(p, num_spans, stream);
    if (dim <= 64) return launch_delta<16, 4>(p, num_spans, stream);
    if (dim <= 128) return launch_delta<16, 8>(p, num_spans, stream);
    return launch_delta<32, 8>(p, num_spans, stream);
}

// out[t, n] = f(sum_r x[t, x_off + r] * w[n, r] + bias[n]) for T rows of x (row stride x_stride elements, float or bf16),
// w [N, R] float or bf16, bias float [N] or null, out [T, N] float or bf16.  mode 0: f = identity; 1: sigmoid;
// 2: exp(-rate[n / per_rate] * softplus(.)), rate float [N / per_rate].
LLB_EXPORT int llb_low_rank_up(const void* x, int x_dtype, long long x_stride, int x_off, int T, int R, const void* w,
                               int w_dtype, int N, const float* bias, int mode, const float* rate, int per_rate,
                               void* out, int out_dtype, cudaStream_t stream) {
    if (T == 0 || N == 0) return 0;
    LLB_REQUIRE(T > 0 && R > 0 && N > 0 && x && w && out, "low_rank_up: bad arguments");
    LLB_REQUIRE(mode >= 0 && mode <= 2 && (mode != 2 || (rate && per_rate > 0)), "low_rank_up: bad mode %d", mode);
    LLB_REQUIRE(R <= 8192, "low_rank_up: %d inputs; at most 8192", R);
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
