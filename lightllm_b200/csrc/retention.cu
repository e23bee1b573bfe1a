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
// (rows d = dg * NR .. dg * NR + NR - 1), in registers; the DG partial sums meet by shuffles.  A block takes one piece
// of one span (up to `chunk` tokens), one head and up to 256 / DG columns, stages 16 rotated q and k rows at a time in
// shared memory (padded with zeros to NR * DG, so the inner loop has no bounds) and walks them token by token with
// 16-byte shared loads.
//
// A long span would leave the GPU to a few warps, so it is cut into pieces that run at the same time, in three passes:
//   local   every piece but a span's last runs the recurrence from a zero state, without outputs, and leaves its
//           contribution A_c = sum_j decay^(n_c - 1 - j) k_j v_j^T in scratch;
//   scan    per span: start_0 = the request's state (zero at position 0), start_c = decay^(n_(c-1)) start_(c-1) + A_(c-1),
//           written over the contributions;
//   out     every piece runs the recurrence from its start state with outputs; a span's last piece writes the
//           request's state slot.
// Spans of one piece (decoding, short portions) take the last pass alone.  Any cutting of a sequence into spans and of
// spans into pieces gives the same recurrence up to the rounding of the float sums.
#include "common.cuh"

namespace {

constexpr int RET_STAGE = 16;      // tokens staged in shared memory at a time

struct RetParams {
    const void* src;          // [T, row_stride]: q, k, v column ranges
    long long row_stride;
    int q_off, k_off, v_off;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* span_slot;
    const int* item_span;     // [items]: the span a piece belongs to
    const int* item_c;        // [items]: which piece of its span
    const int* span_first;    // [spans]: index of a span's first piece (= its place in scratch)
    const float* decay;       // [H]
    const float* inv_freq;    // [rotary_dim / 2]
    int rotary_dim, interleaved;
    float k_scale;
    float* state;             // [slots, H, dim, vdim]
    float* scratch;           // [items, H, dim, vdim] (only read or written for spans of several pieces)
    float* out;               // [T, H, vdim] float
    int H, dim, vdim, EV, chunk, mode;
};

enum { RET_LOCAL = 1, RET_OUT = 3 };

template <typename T, int NR, int DG, int MODE>
__global__ void __launch_bounds__(256) retention_kernel(RetParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int PADF = DG > 1 ? 4 : 0;                 // keeps the DG threads of a column on different banks
    constexpr int DPAD = DG * (NR + PADF);
    const int item = blockIdx.x, h = blockIdx.y;
    const int span = p.item_span[item], c = p.item_c[item];
    const int dim = p.dim, vdim = p.vdim;
    const int slen = p.span_len[span];
    const int pieces = (slen + p.chunk - 1) / p.chunk;
    const bool last = c == pieces - 1;
    if (MODE == RET_LOCAL && last) return;               // the last piece's contribution is never needed
    float* qs = sm;                          // [RET_STAGE][DPAD]
    float* ks = qs + RET_STAGE * DPAD;       // [RET_STAGE][DPAD]
    float* vs = ks + RET_STAGE * DPAD;       // [RET_STAGE][EV]
    const int dg = threadIdx.x % DG, el = threadIdx.x / DG;
    const int e = blockIdx.z * p.EV + el;
    const bool live = el < p.EV && e < vdim;
    const int t0 = c * p.chunk;
    const int len = min(p.chunk, slen - t0);
    const int row0 = p.span_row[span] + t0, pos0 = p.span_pos[span] + t0;
    const float decay = p.decay[h];
    const size_t plane = (size_t)dim * vdim;
    float* slot = p.state + ((size_t)p.span_slot[span] * p.H + h) * plane;
    const T* src = (const T*)p.src;

    // start state: zero (local pass; a request's first token), the request's slot, or what the scan left for this piece
    const float* from = nullptr;
    if (MODE == RET_OUT) {
        if (pieces > 1) from = p.scratch + ((size_t)item * p.H + h) * plane;
        else if (pos0 > 0) from = slot;
    }
    float S[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = dg * NR + j;
        S[j] = (from != nullptr && live && d < dim) ? from[(size_t)d * vdim + e] : 0.0f;
    }
    for (int i = threadIdx.x; i < 2 * RET_STAGE * DPAD; i += blockDim.x) sm[i] = 0.0f;     // the padding stays zero
    const int half = p.rotary_dim / 2;
    const int per_row = dim - half;          // rotated pairs + pass-through singles
    auto at = [](int d) { return (d / NR) * (NR + PADF) + d % NR; };
    for (int c0 = 0; c0 < len; c0 += RET_STAGE) {
        const int n = min(RET_STAGE, len - c0);
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
                const float cs = cosf(angle), sn = sinf(angle);
                float a, b;
                if (MODE == RET_OUT) {           // the local pass makes no outputs and needs no q
                    a = llb_to_float(qr[ia]);
                    b = llb_to_float(qr[ib]);
                    qs[tl * DPAD + at(ia)] = a * cs - b * sn;
                    qs[tl * DPAD + at(ib)] = b * cs + a * sn;
                }
                a = llb_to_float(kr[ia]);
                b = llb_to_float(kr[ib]);
                ks[tl * DPAD + at(ia)] = (a * cs - b * sn) * p.k_scale;
                ks[tl * DPAD + at(ib)] = (b * cs + a * sn) * p.k_scale;
            } else {
                const int d = p.rotary_dim + (j - half);
                if (MODE == RET_OUT) qs[tl * DPAD + at(d)] = llb_to_float(qr[d]);
                ks[tl * DPAD + at(d)] = llb_to_float(kr[d]) * p.k_scale;
            }
        }
        for (int it = threadIdx.x; it < n * p.EV; it += blockDim.x) {
            const int tl = it / p.EV, cc = it - tl * p.EV;
            const int ee = blockIdx.z * p.EV + cc;
            vs[it] = ee < vdim ? llb_to_float(src[(size_t)(row0 + c0 + tl) * p.row_stride + p.v_off + (size_t)h * vdim + ee]) : 0.0f;
        }
        __syncthreads();
        for (int tl = 0; tl < n; ++tl) {
            const float vv = el < p.EV ? vs[tl * p.EV + el] : 0.0f;
            const float4* kq = reinterpret_cast<const float4*>(ks + tl * DPAD + dg * (NR + PADF));
            const float4* qq = reinterpret_cast<const float4*>(qs + tl * DPAD + dg * (NR + PADF));
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int j = 0; j < NR; j += 4) {
                const float4 k4 = kq[j >> 2];
                S[j] = fmaf(decay, S[j], k4.x * vv);
                S[j + 1] = fmaf(decay, S[j + 1], k4.y * vv);
                S[j + 2] = fmaf(decay, S[j + 2], k4.z * vv);
                S[j + 3] = fmaf(decay, S[j + 3], k4.w * vv);
                if (MODE == RET_OUT) {
                    const float4 q4 = qq[j >> 2];
                    a0 = fmaf(S[j], q4.x, a0);
                    a1 = fmaf(S[j + 1], q4.y, a1);
                    a2 = fmaf(S[j + 2], q4.z, a2);
                    a3 = fmaf(S[j + 3], q4.w, a3);
                }
            }
            if (MODE == RET_OUT) {
                float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
                for (int o = 1; o < DG; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (live && dg == 0) p.out[((size_t)(row0 + c0 + tl) * p.H + h) * vdim + e] = acc;
            }
        }
    }
    if (!live) return;
    float* to = nullptr;
    if (MODE == RET_LOCAL) to = p.scratch + ((size_t)(item + 1) * p.H + h) * plane;     // the next piece's place
    else if (last) to = slot;
    if (to != nullptr) {
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int d = dg * NR + j;
            if (d < dim) to[(size_t)d * vdim + e] = S[j];
        }
    }
}

// start_0 = the request's state (zero at position 0); start_c = decay^(tokens of piece c-1) * start_(c-1) + A_(c-1).
// One thread per element of a head's state; the pieces of a span one after the other.
__global__ void __launch_bounds__(256) retention_scan_kernel(RetParams p) {
    const int span = blockIdx.x, h = blockIdx.y;
    const int slen = p.span_len[span];
    const int pieces = (slen + p.chunk - 1) / p.chunk;
    if (pieces <= 1) return;
    const size_t plane = (size_t)p.dim * p.vdim;
    const float* slot = p.state + ((size_t)p.span_slot[span] * p.H + h) * plane;
    const bool fresh = p.span_pos[span] == 0;
    const float step = powf(p.decay[h], (float)p.chunk);          // every piece but the last has `chunk` tokens
    const size_t first = (size_t)p.span_first[span];
    const size_t stride = (size_t)p.H * plane;          // from one piece's place to the next
    for (size_t i = (size_t)blockIdx.z * blockDim.x + threadIdx.x; i < plane; i += (size_t)gridDim.z * blockDim.x) {
        float s = fresh ? 0.0f : slot[i];
        float* at = p.scratch + (first * p.H + h) * plane + i;
        at[0] = s;
        // eight pieces' contributions are requested together; only the additions wait for one another
        for (int c = 1; c < pieces; c += 8) {
            float a[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) a[u] = c + u < pieces ? at[(size_t)(c + u) * stride] : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                s = fmaf(step, s, a[u]);
                a[u] = s;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (c + u < pieces) at[(size_t)(c + u) * stride] = a[u];
        }
    }
}

template <typename T, int NR, int DG>
int launch_retention_as(const RetParams& p, int num_items, cudaStream_t stream) {
    constexpr int PADF = DG > 1 ? 4 : 0;
    dim3 grid(num_items, p.H, llb_ceil_div(p.vdim, p.EV));
    const int threads = ((p.EV * DG + 31) / 32) * 32;
    const size_t smem = ((size_t)2 * RET_STAGE * DG * (NR + PADF) + (size_t)RET_STAGE * p.EV) * sizeof(float);
    if (p.mode == RET_LOCAL) retention_kernel<T, NR, DG, RET_LOCAL><<<grid, threads, smem, stream>>>(p);
    else retention_kernel<T, NR, DG, RET_OUT><<<grid, threads, smem, stream>>>(p);
    return llb_check_launch("retention");
}

template <typename T>
int launch_retention(const RetParams& p, int num_items, cudaStream_t stream) {
    if (p.dim <= 16) return launch_retention_as<T, 16, 1>(p, num_items, stream);
    if (p.dim <= 32) return launch_retention_as<T, 32, 1>(p, num_items, stream);
    if (p.dim <= 64) return launch_retention_as<T, 64, 1>(p, num_items, stream);
    if (p.dim <= 128) return launch_retention_as<T, 64, 2>(p, num_items, stream);
    if (p.dim <= 256) return launch_retention_as<T, 64, 4>(p, num_items, stream);
    return launch_retention_as<T, 64, 8>(p, num_items, stream);
}

}  // namespace

// src: row t at src + t * row_stride with q [H, dim] at q_off, k [H, dim] at k_off, v [H, vdim] at v_off (dtype);
// spans as the step describes them (first row, length, first position, state slot); the spans cut into pieces of
// `chunk` tokens: item_span / item_c [num_items] name each piece (span, index within it; a span's pieces are
// consecutive items), span_first [num_spans] the index of a span's first piece; decay [H] float;
// inv_freq [rotary_dim/2] float (unused when rotary_dim == 0); k_scale multiplies k after the rotation;
// state float [slots, H, dim, vdim]; scratch float [num_items, H, dim, vdim], needed (multi != 0) when a span has
// several pieces; out float [T, H, vdim].
LLB_EXPORT int llb_retention(const void* src, int dtype, long long row_stride, int q_off, int k_off, int v_off,
                             const int* span_row, const int* span_len, const int* span_pos, const int* span_slot,
                             int num_spans, const int* item_span, const int* item_c, const int* span_first, int num_items,
                             int chunk, int multi, int H, int dim, int vdim, const float* decay, const float* inv_freq,
                             int rotary_dim, int interleaved, float k_scale, float* state, float* scratch, float* out,
                             cudaStream_t stream) {
    if (num_spans == 0) return 0;
    LLB_REQUIRE(num_spans > 0 && num_items >= num_spans && chunk > 0 && H > 0 && dim > 0 && vdim > 0 && src && state &&
                out && decay && item_span && item_c && span_first, "retention: bad arguments");
    LLB_REQUIRE(!multi || scratch != nullptr, "retention: spans of several pieces need scratch");
    LLB_REQUIRE(H <= 65535 && dim <= 512, "retention: at most 65535 heads of at most 512 dimensions");
    LLB_REQUIRE(rotary_dim >= 0 && rotary_dim <= dim && rotary_dim % 2 == 0,
                "retention: rotary_dim %d must be even and at most %d", rotary_dim, dim);
    LLB_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "retention: inv_freq is null");
    RetParams p;
    p.src = src; p.row_stride = row_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
    p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.item_span = item_span; p.item_c = item_c; p.span_first = span_first;
    p.decay = decay; p.inv_freq = inv_freq; p.rotary_dim = rotary_dim; p.interleaved = interleaved ? 1 : 0;
    p.k_scale = k_scale; p.state = state; p.scratch = scratch; p.out = out; p.H = H; p.dim = dim; p.vdim = vdim;
    p.chunk = chunk;
    // a thread keeps at most 64 rows of its column: DG threads share a column of more
    const int DG = dim <= 64 ? 1 : dim <= 128 ? 2 : dim <= 256 ? 4 : 8;
    const int per_block = 256 / DG;
    p.EV = vdim < per_block ? vdim : per_block;
    LLB_REQUIRE(llb_ceil_div(vdim, p.EV) <= 65535, "retention: too many columns");
    int rc = 0;
    for (int pass = multi ? 0 : 2; pass < 3 && rc == 0; ++pass) {
        if (pass == 1) {
            const size_t plane = (size_t)dim * vdim;
            int z = (int)((plane + 255) / 256);
            if (z > 64) z = 64;
            retention_scan_kernel<<<dim3(num_spans, H, z), 256, 0, stream>>>(p);
            rc = llb_check_launch("retention_scan");
            continue;
        }
        p.mode = pass == 0 ? RET_LOCAL : RET_OUT;
        if (dtype == LLB_F32) rc = launch_retention<float>(p, num_items, stream);
        else if (dtype == LLB_BF16) rc = launch_retention<__nv_bfloat16>(p, num_items, stream);
        else return llb_fail("retention: unknown dtype %d", dtype);
    }
    return rc;
}
