// Layer normalisation with weight and (optionally) bias over rows of a float stream, optionally only over a list of rows, and
// optionally added into a float destination (a norm on a branch's output: h += LN(branch) in one pass).
//
//     mean = sum_d x_d / D;  var = sum_d (x_d - mean)^2 / D;  y_d = (x_d - mean) / sqrt(var + eps) * w_d + b_d
//
// All statistics are float; the variance is taken from the deviations (second pass over the row, which stays in
// registers when it fits), not from E[x^2] - mean^2.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* part, float* total) {
    v = llb_warp_sum(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.0f;
        t = llb_warp_sum(t);
        if (threadIdx.x == 0) *total = t;
    }
    __syncthreads();
    const float r = *total;
    __syncthreads();
    return r;
}

template <typename TW, typename TO, int PER_THREAD, bool ACCUMULATE>
__global__ void __launch_bounds__(256) layernorm_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                                        const TW* __restrict__ b, TO* __restrict__ out,
                                                        const int* __restrict__ rows, int D, float eps,
                                                        __nv_bfloat16* __restrict__ copy) {
    __shared__ float part[32];
    __shared__ float total;
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    TO* o = out + (size_t)r * D;
    float v[PER_THREAD > 0 ? PER_THREAD : 1];
    float s = 0.0f;
    if (PER_THREAD > 0) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            v[i] = d < D ? xr[d] : 0.0f;
            s += v[i];
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) s += xr[d];
    }
    const float mean = block_sum(s, part, &total) / (float)D;
    float q = 0.0f;
    if (PER_THREAD > 0) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            const float c = d < D ? v[i] - mean : 0.0f;
            q += c * c;
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const float c = xr[d] - mean;
            q += c * c;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(q, part, &total) / (float)D + eps);
    if (PER_THREAD > 0) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d < D) {
                float y = (v[i] - mean) * inv * llb_to_float(w[d]) + (b ? llb_to_float(b[d]) : 0.0f);
                if (ACCUMULATE) y += llb_to_float(o[d]);
                o[d] = llb_from_float<TO>(y);
                if (copy) copy[(size_t)r * D + d] = __float2bfloat16_rn(y);
            }
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float y = (xr[d] - mean) * inv * llb_to_float(w[d]) + (b ? llb_to_float(b[d]) : 0.0f);
            if (ACCUMULATE) y += llb_to_float(o[d]);
            o[d] = llb_from_float<TO>(y);
            if (copy) copy[(size_t)r * D + d] = __float2bfloat16_rn(y);
        }
    }
}

__device__ __forceinline__ float4 ln_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ln_load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, c.x, c.y);
}
__device__ __forceinline__ void ln_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ln_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), c = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&c));
}

// One warp per row of a width that is a multiple of 4 and at most 128 * NV: the row stays in registers as NV float4 a
// lane, both sums need shuffles only, and every access is 16 (float) or 8 (bf16) bytes wide.
template <typename TW, typename TO, int NV, bool ACCUMULATE>
__global__ void __launch_bounds__(256) layernorm_warp_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                                             const TW* __restrict__ b, TO* __restrict__ out,
                                                             const int* __restrict__ rows, int R, int D, float eps,
                                                             __nv_bfloat16* __restrict__ copy) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float4 v[NV];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        v[i] = d < D ? ln_load4(xr + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = llb_warp_sum(s) / (float)D;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (d < D) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            q += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    const float inv = 1.0f / sqrtf(llb_warp_sum(q) / (float)D + eps);
    TO* o = out + (size_t)r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (d < D) {
            const float4 g = ln_load4(w + d), c = b ? ln_load4(b + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 y = make_float4(v[i].x * inv * g.x + c.x, v[i].y * inv * g.y + c.y, v[i].z * inv * g.z + c.z,
                                   v[i].w * inv * g.w + c.w);
            if (ACCUMULATE) {
                const float4 old = ln_load4(o + d);
                y.x += old.x; y.y += old.y; y.z += old.z; y.w += old.w;
            }
            ln_store4(o + d, y);
            if (copy) ln_store4(copy + (size_t)r * D + d, y);
        }
    }
}

template <typename TW, typename TO, bool ACC>
int launch_ln(const float* x, const void* w, const void* b, void* out, const int* rows, int R, int D, float eps,
              __nv_bfloat16* copy, cudaStream_t s) {
    const int threads = 256;
    const bool aligned = D % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)b % 16 == 0 &&
                         (uintptr_t)out % 16 == 0 && (uintptr_t)copy % 8 == 0;
    if (aligned && D <= 128 * 8)
        layernorm_warp_kernel<TW, TO, 8, ACC><<<(R + 7) / 8, threads, 0, s>>>(x, (const TW*)w, (const TW*)b, (TO*)out, rows,
                                                                              R, D, eps, copy);
    else if (aligned && D <= 128 * 16)
        layernorm_warp_kernel<TW, TO, 16, ACC><<<(R + 7) / 8, threads, 0, s>>>(x, (const TW*)w, (const TW*)b, (TO*)out, rows,
                                                                               R, D, eps, copy);
    else if (D <= threads * 4)
        layernorm_kernel<TW, TO, 4, ACC><<<R, threads, 0, s>>>(x, (const TW*)w, (const TW*)b, (TO*)out, rows, D, eps, copy);
    else if (D <= threads * 16)
        layernorm_kernel<TW, TO, 16, ACC><<<R, threads, 0, s>>>(x, (const TW*)w, (const TW*)b, (TO*)out, rows, D, eps, copy);
    else
        layernorm_kernel<TW, TO, 0, ACC><<<R, threads, 0, s>>>(x, (const TW*)w, (const TW*)b, (TO*)out, rows, D, eps, copy);
    return llb_check_launch("layernorm");
}

template <typename TW>
int dispatch_ln(int out_dtype, int accumulate, const float* x, const void* w, const void* b, void* out, const int* rows,
                int R, int D, float eps, __nv_bfloat16* copy, cudaStream_t s) {
    if (out_dtype == LLB_F32)
        return accumulate ? launch_ln<TW, float, true>(x, w, b, out, rows, R, D, eps, copy, s)
                          : launch_ln<TW, float, false>(x, w, b, out, rows, R, D, eps, copy, s);
    if (out_dtype == LLB_BF16)
        return accumulate ? launch_ln<TW, __nv_bfloat16, true>(x, w, b, out, rows, R, D, eps, copy, s)
                          : launch_ln<TW, __nv_bfloat16, false>(x, w, b, out, rows, R, D, eps, copy, s);
    return llb_fail("layernorm: unknown output dtype %d", out_dtype);
}

}  // namespace

// x float [*, D]; w, b [D] (float or bf16, the same for both; b may be null: no bias); out [R, D]; rows: R source rows of x or null for
// rows 0..R-1; accumulate != 0: out += LN(x) (out must not be x); copy: bf16 [R, D] or null, receives what was
// written to out (the updated stream, for the next branch's projections).
LLB_EXPORT int llb_layernorm(const float* x, const void* w, const void* b, int w_dtype, void* out, int out_dtype,
                             const int* rows, int R, int D, float eps, int accumulate, void* copy, cudaStream_t stream) {
    if (R == 0) return 0;
    LLB_REQUIRE(R > 0 && D > 0 && x && w && out, "layernorm: bad arguments R=%d D=%d", R, D);
    __nv_bfloat16* c = (__nv_bfloat16*)copy;
    if (w_dtype == LLB_F32) return dispatch_ln<float>(out_dtype, accumulate, x, w, b, out, rows, R, D, eps, c, stream);
    if (w_dtype == LLB_BF16) return dispatch_ln<__nv_bfloat16>(out_dtype, accumulate, x, w, b, out, rows, R, D, eps, c, stream);
    return llb_fail("layernorm: unknown weight dtype %d", w_dtype);
}
