// Routing of a mixture of experts, in float: logits z = W_r x, scores by a sigmoid or a softmax over the experts, the
// `top` experts with the largest choice scores (score + an optional per-expert correction that takes part in the choice
// only), weights = the chosen experts' scores (optionally renormalised to sum 1) times `scale`.
//
// One warp per token.  The result is written twice: as lists (`ids`, `weights` [T, top], in the order of the choice) and
// as a dense row of weights over all experts (`dense` [T, E], zero for the experts not chosen), which is what the
// contraction-shaped expert path multiplies the experts' activations by.
#include "common.cuh"

namespace {

constexpr int MOE_MAX_EXPERTS = 512;

template <typename TX>
__global__ void __launch_bounds__(128) moe_route_kernel(const TX* __restrict__ x, const float* __restrict__ w,
                                                        const float* __restrict__ correction, int T, int D, int E, int top,
                                                        int softmax, int renorm, float scale, int* __restrict__ ids,
                                                        float* __restrict__ weights, float* __restrict__ dense) {
    extern __shared__ float sm[];                // per warp: score [E], choice [E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* score = sm + (size_t)warp * 2 * E;
    float* choice = score + E;
    const TX* xr = x + (size_t)t * D;
    for (int e = 0; e < E; ++e) {
        const float* wr = w + (size_t)e * D;
        float acc = 0.0f;
        for (int d = lane; d < D; d += 32) acc = fmaf(llb_to_float(xr[d]), wr[d], acc);
        acc = llb_warp_sum(acc);
        if (lane == 0) score[e] = acc;
    }
    __syncwarp();
    if (softmax) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, score[e]);
        m = llb_warp_max(m);
        float s = 0.0f;
        for (int e = lane; e < E; e += 32) s += expf(score[e] - m);
        s = llb_warp_sum(s);
        for (int e = lane; e < E; e += 32) score[e] = expf(score[e] - m) / s;
    } else {
        for (int e = lane; e < E; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        choice[e] = score[e] + (correction ? correction[e] : 0.0f);
        dense[(size_t)t * E + e] = 0.0f;
    }
    __syncwarp();
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = E;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; arg = e; }          // the lowest index among equals of a lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= E) arg = 0;                            // only when every score is NaN
        const float s = score[arg];
        total += s;
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = s;
            choice[arg] = -INFINITY;
        }
        __syncwarp();
    }
    const float mul = renorm ? scale / total : scale;
    __syncwarp();
    if (lane < top || top > 32) {
        for (int k = lane; k < top; k += 32) {
            const float wgt = weights[(size_t)t * top + k] * mul;
            weights[(size_t)t * top + k] = wgt;
            dense[(size_t)t * E + ids[(size_t)t * top + k]] = wgt;
        }
    }
}

// act[t, e * F + j] *= dense[t, e]; exactly zero where the expert was not chosen, whatever the activation holds.
template <typename TA>
__global__ void moe_scale_kernel(TA* __restrict__ act, const float* __restrict__ dense, long long n, int E, int F) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long row = (long long)E * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long t = i / row;
        const int e = (int)((i - t * row) / F);
        const float wgt = dense[t * E + e];
        act[i] = wgt == 0.0f ? llb_from_float<TA>(0.0f) : llb_from_float<TA>(llb_to_float(act[i]) * wgt);
    }
}

// The (token, chosen expert) pairs in expert order, every expert's pairs padded to whole tiles of `align` rows: slot[i] is
// the row of pair i (token i / top, its choice i % top), tile_group[m] the expert of tile m (0 for tiles behind the last
// expert's).  One block: counts in shared memory, a serial walk over the experts, then a cursor per expert.  Which of an
// expert's rows a pair gets depends on the order of the atomic adds; no result depends on it.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int pairs, int E, int align, int max_tiles,
                                                        int* __restrict__ slot, int* __restrict__ tile_group) {
    extern __shared__ int sh[];                  // count [E], cursor [E]
    int* count = sh;
    int* cursor = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = tile * align;
            const int n = (count[e] + align - 1) / align;
            for (int j = 0; j < n && tile < max_tiles; ++j) tile_group[tile++] = e;
        }
        while (tile < max_tiles) tile_group[tile++] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) slot[i] = atomicAdd(&cursor[ids[i]], 1);
}

// xs[slot[i], :] = x[i / top, :]
template <typename TX>
__global__ void __launch_bounds__(128) moe_gather_kernel(const TX* __restrict__ x, const int* __restrict__ slot, int top, int D,
                                                         TX* __restrict__ xs) {
    const int i = blockIdx.x;
    const TX* src = x + (size_t)(i / top) * D;
    TX* dst = xs + (size_t)slot[i] * D;
    constexpr int V = 16 / sizeof(TX);
    if (D % V == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xs % 16 == 0) {
        for (int d = threadIdx.x; d < D / V; d += blockDim.x)
            reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(src)[d];
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
    }
}

// residual[t, :] += sum_k weights[t, k] * y[slot[t * top + k], :], the choices added in their order
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ slot,
                                                          const float* __restrict__ weights, int top, int D,
                                                          float* __restrict__ residual) {
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int k = 0; k < top; ++k) acc = fmaf(weights[(size_t)t * top + k], y[(size_t)slot[(size_t)t * top + k] * D + d], acc);
        residual[(size_t)t * D + d] += acc;
    }
}

}  // namespace

// ids int [T * top] -> slot int [T * top], tile_group int [max_tiles] (see moe_sort_kernel); max_tiles >= T * top / align + E.
LLB_EXPORT int llb_moe_sort(const int* ids, int pairs, int E, int align, int max_tiles, int* slot, int* tile_group,
                            cudaStream_t stream) {
    if (pairs == 0) return 0;
    LLB_REQUIRE(pairs > 0 && E > 0 && E <= 4096 && align > 0 && ids && slot && tile_group, "moe_sort: bad arguments");
    LLB_REQUIRE(max_tiles >= pairs / align + E, "moe_sort: %d tiles cannot hold %d pairs of %d experts", max_tiles, pairs, E);
    moe_sort_kernel<<<1, 1024, 2 * E * sizeof(int), stream>>>(ids, pairs, E, align, max_tiles, slot, tile_group);
    return llb_check_launch("moe_sort");
}

// x [T, D] -> xs [rows, D] (same dtype): row slot[i] of xs is row i / top of x, for the T * top pairs.
LLB_EXPORT int llb_moe_gather(const void* x, int dtype, const int* slot, int pairs, int top, int D, void* xs,
                              cudaStream_t stream) {
    if (pairs == 0) return 0;
    LLB_REQUIRE(pairs > 0 && top > 0 && D > 0 && x && slot && xs, "moe_gather: bad arguments");
    if (dtype == LLB_F32) moe_gather_kernel<float><<<pairs, 128, 0, stream>>>((const float*)x, slot, top, D, (float*)xs);
    else if (dtype == LLB_BF16)
        moe_gather_kernel<__nv_bfloat16><<<pairs, 128, 0, stream>>>((const __nv_bfloat16*)x, slot, top, D, (__nv_bfloat16*)xs);
    else return llb_fail("moe_gather: unknown dtype %d", dtype);
    return llb_check_launch("moe_gather");
}

// y float [rows, D], slot int [T * top], weights float [T, top], residual float [T, D] += the weighted rows.
LLB_EXPORT int llb_moe_combine(const float* y, const int* slot, const float* weights, int T, int top, int D, float* residual,
                               cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && top > 0 && D > 0 && y && slot && weights && residual, "moe_combine: bad arguments");
    moe_combine_kernel<<<T, 256, 0, stream>>>(y, slot, weights, top, D, residual);
    return llb_check_launch("moe_combine");
}

// x [T, D] float or bf16; w float [E, D]; correction float [E] or null; ids int [T, top]; weights float [T, top];
// dense float [T, E].  softmax != 0: scores by a softmax over the experts, else by a sigmoid of each logit;
// renorm != 0: the chosen scores are divided by their sum before `scale`.
LLB_EXPORT int llb_moe_route(const void* x, int x_dtype, const float* w, const float* correction, int T, int D, int E,
                             int top, int softmax, int renorm, float scale, int* ids, float* weights, float* dense,
                             cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && x && w && ids && weights && dense, "moe_route: bad arguments");
    LLB_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "moe_route: top %d of %d experts (at most %d)", top, E,
                MOE_MAX_EXPERTS);
    const int warps = 4;
    const size_t smem = (size_t)warps * 2 * E * sizeof(float);
    const unsigned blocks = (unsigned)((T + warps - 1) / warps);
    if (x_dtype == LLB_F32)
        moe_route_kernel<float><<<blocks, warps * 32, smem, stream>>>((const float*)x, w, correction, T, D, E, top, softmax,
                                                                      renorm, scale, ids, weights, dense);
    else if (x_dtype == LLB_BF16)
        moe_route_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>((const __nv_bfloat16*)x, w, correction, T, D, E,
                                                                              top, softmax, renorm, scale, ids, weights, dense);
    else
        return llb_fail("moe_route: unknown dtype %d", x_dtype);
    return llb_check_launch("moe_route");
}

// act [T, E * F] (float or bf16), in place: the activations of expert e of row t times dense[t, e].
LLB_EXPORT int llb_moe_scale(void* act, int dtype, const float* dense, int T, int E, int F, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && E > 0 && F > 0 && act && dense, "moe_scale: bad arguments");
    const long long n = (long long)T * E * F;
    const int blocks = (int)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
    if (dtype == LLB_F32) moe_scale_kernel<float><<<blocks, 256, 0, stream>>>((float*)act, dense, n, E, F);
    else if (dtype == LLB_BF16) moe_scale_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)act, dense, n, E, F);
    else return llb_fail("moe_scale: unknown dtype %d", dtype);
    return llb_check_launch("moe_scale");
}
