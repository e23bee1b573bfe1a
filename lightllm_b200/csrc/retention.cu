// Retention: linear attention with a fixed decay per head, no softmax and no denominator, as a recurrence over a
// per-request state that lives in float:
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T          S [dim, vdim] per head, zero before a request's first token
//     o_t = S_t^T q_t
//
// q and k are rotated by position inside the kernel (pairs (i, i + rotary_dim/2) or (2i, 2i+1), angle = pos * inv_freq[i]),
// k is scaled after the rotation; everything from the rotation on is float whatever the dtype of the projections.
//
// The columns of S are independent (o_t[e] = sum_d S[d, e] q_t[d]), so a thread owns one column e, or a DG-th of it
// (rows d = dg, dg + DG, ...), in registers for a whole span of tokens; the DG partial sums meet by shuffles.  A block
// takes one span, one head and up to 256 / DG columns, stages chunks of rotated q and k rows in shared memory and walks
// them token by token.  The state is read from the request's slot when the span does not start the request, and
// written back at its end, so any cutting of a sequence into spans gives the same recurrence.
#include "common.cuh"

namespace {

constexpr int RET_CHUNK = 16;

struct RetParams {
    const void* src;          // [T, row_stride]: q, k, v column ranges
    long long row_stride;
    int q_off, k_off, v_off;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* span_slot;
    const float* decay;       // [H]
    const float* inv_freq;    // [rotary_dim / 2]
    int rotary_dim, interleaved;
    float k_scale;
    float* state;             // [slots, H, dim, vdim]
    float* out;               // [T, H, vdim] float
    int H, dim, vdim, DG, EV;
};

template <typename T, int NR>
__global__ void __launch_bounds__(256) retention_kernel(RetParams p) {
    extern __shared__ float sm[];
    const int span = blockIdx.x, h = blockIdx.y;
    const int dim = p.dim, vdim = p.vdim, DG = p.DG;
    float* qs = sm;                          // [RET_CHUNK][dim]
    float* ks = qs + RET_CHUNK * dim;        // [RET_CHUNK][dim]
    float* vs = ks + RET_CHUNK * dim;        // [RET_CHUNK][EV]
    const int dg = threadIdx.x % DG, el = threadIdx.x / DG;
    const int e = blockIdx.z * p.EV + el;
    const bool live = el < p.EV && e < vdim;
    const int row0 = p.span_row[span], len = p.span_len[span], pos0 = p.span_pos[span];
    const float decay = p.decay[h];
    float* st = p.state + (((size_t)p.span_slot[span] * p.H + h) * dim) * vdim;
    const T* src = (const T*)p.src;

    float S[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = dg + DG * j;
        S[j] = (pos0 > 0 && live && d < dim) ? st[(size_t)d * vdim + e] : 0.0f;
    }
    const int half = p.rotary_dim / 2;
    const int per_row = dim - half;          // rotated pairs + pass-through singles
    for (int c0 = 0; c0 < len; c0 += RET_CHUNK) {
        const int n = min(RET_CHUNK, len - c0);
        __syncthreads();
        for (int it = threadIdx.x; it < n * per_row; it += blockDim.x) {
            const int tl = it / per_row, j = it - tl * per_row;
            const T* row = src + (size_t)(row0 + c0 + tl) * p.row_stride;
            const T* qr = row + p.q_off + (size_t)h * dim;
            const T* kr = row + p.k_off + (size_t)h * dim;
            if (j < half) {
                const int ia = p.interleaved ? 2 * j : j;
                const int ib = p.interleaved ? 2 * j + 1 : j + half;
                const float angle = (float)(pos0 + c0 + tl) * p.inv_freq[j];
                const float c = cosf(angle), s = sinf(angle);
                float a = llb_to_float(qr[ia]), b = llb_to_float(qr[ib]);
                qs[tl * dim + ia] = a * c - b * s;
                qs[tl * dim + ib] = b * c + a * s;
                a = llb_to_float(kr[ia]);
                b = llb_to_float(kr[ib]);
                ks[tl * dim + ia] = (a * c - b * s) * p.k_scale;
                ks[tl * dim + ib] = (b * c + a * s) * p.k_scale;
            } else {
                const int d = p.rotary_dim + (j - half);
                qs[tl * dim + d] = llb_to_float(qr[d]);
                ks[tl * dim + d] = llb_to_float(kr[d]) * p.k_scale;
            }
        }
        for (int it = threadIdx.x; it < n * p.EV; it += blockDim.x) {
            const int tl = it / p.EV, c = it - tl * p.EV;
            const int ee = blockIdx.z * p.EV + c;
            vs[it] = ee < vdim ? llb_to_float(src[(size_t)(row0 + c0 + tl) * p.row_stride + p.v_off + (size_t)h * vdim + ee]) : 0.0f;
        }
        __syncthreads();
        for (int tl = 0; tl < n; ++tl) {
            const float vv = el < p.EV ? vs[tl * p.EV + el] : 0.0f;
            const float* kq = ks + tl * dim;
            const float* qq = qs + tl * dim;
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < NR; ++j) {
                const int d = dg + DG * j;
                if (d < dim) {
                    S[j] = fmaf(decay, S[j], kq[d] * vv);
                    acc = fmaf(S[j], qq[d], acc);
                }
            }
            for (int o = 1; o < DG; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && dg == 0) p.out[((size_t)(row0 + c0 + tl) * p.H + h) * vdim + e] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int d = dg + DG * j;
            if (d < dim) st[(size_t)d * vdim + e] = S[j];
        }
    }
}

template <typename T>
int launch_retention(const RetParams& p, int num_spans, cudaStream_t stream) {
    const int columns = llb_ceil_div(p.vdim, p.EV);
    dim3 grid(num_spans, p.H, columns);
    const int threads = ((p.EV * p.DG + 31) / 32) * 32;
    const size_t smem = ((size_t)2 * RET_CHUNK * p.dim + (size_t)RET_CHUNK * p.EV) * sizeof(float);
    const int nr = llb_ceil_div(p.dim, p.DG);
    if (nr <= 16) retention_kernel<T, 16><<<grid, threads, smem, stream>>>(p);
    else if (nr <= 32) retention_kernel<T, 32><<<grid, threads, smem, stream>>>(p);
    else retention_kernel<T, 64><<<grid, threads, smem, stream>>>(p);
    return llb_check_launch("retention");
}

}  // namespace

// src: row t at src + t * row_stride with q [H, dim] at q_off, k [H, dim] at k_off, v [H, vdim] at v_off (dtype);
// spans as the step describes them (first row, length, first position, state slot); decay [H] float;
// inv_freq [rotary_dim/2] float (unused when rotary_dim == 0); k_scale multiplies k after the rotation;
// state float [slots, H, dim, vdim]; out float [T, H, vdim].
LLB_EXPORT int llb_retention(const void* src, int dtype, long long row_stride, int q_off, int k_off, int v_off,
                             const int* span_row, const int* span_len, const int* span_pos, const int* span_slot,
                             int num_spans, int H, int dim, int vdim, const float* decay, const float* inv_freq,
                             int rotary_dim, int interleaved, float k_scale, float* state, float* out,
                             cudaStream_t stream) {
    if (num_spans == 0) return 0;
    LLB_REQUIRE(num_spans > 0 && H > 0 && dim > 0 && vdim > 0 && src && state && out && decay, "retention: bad arguments");
    LLB_REQUIRE(H <= 65535 && dim <= 512, "retention: at most 65535 heads of at most 512 dimensions");
    LLB_REQUIRE(rotary_dim >= 0 && rotary_dim <= dim && rotary_dim % 2 == 0,
                "retention: rotary_dim %d must be even and at most %d", rotary_dim, dim);
    LLB_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "retention: inv_freq is null");
    RetParams p;
    p.src = src; p.row_stride = row_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
    p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.decay = decay; p.inv_freq = inv_freq; p.rotary_dim = rotary_dim; p.interleaved = interleaved ? 1 : 0;
    p.k_scale = k_scale; p.state = state; p.out = out; p.H = H; p.dim = dim; p.vdim = vdim;
    // a thread keeps at most 64 rows of its column: DG threads share a column of more
    p.DG = dim <= 64 ? 1 : dim <= 128 ? 2 : dim <= 256 ? 4 : 8;
    const int per_block = 256 / p.DG;
    p.EV = vdim < per_block ? vdim : per_block;
    LLB_REQUIRE(llb_ceil_div(vdim, p.EV) <= 65535, "retention: too many columns");
    if (dtype == LLB_F32) return launch_retention<float>(p, num_spans, stream);
    if (dtype == LLB_BF16) return launch_retention<__nv_bfloat16>(p, num_spans, stream);
    return llb_fail("retention: unknown dtype %d", dtype);
}
