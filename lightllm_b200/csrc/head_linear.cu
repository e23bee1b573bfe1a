// A contraction per head: out[t, h, o] = sum_i x[t, h, i] * w[h, o, i], for projections that differ from head to head
// (the up-projections of a shared latent folded onto the query and the output).  Float accumulation; x, w and out
// float or bf16.  x may be a column range of a wider row.
#include "common.cuh"

namespace {

constexpr int HL_ROWS = 16;     // tokens per block

template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ x, long long x_stride, int x_off,
                                                          const T* __restrict__ w, T* __restrict__ out, int Tn, int H,
                                                          int in, int on) {
    extern __shared__ float xs[];          // [HL_ROWS][in]
    const int t0 = blockIdx.x * HL_ROWS, h = blockIdx.y;
    const int rows = min(HL_ROWS, Tn - t0);
    for (int i = threadIdx.x; i < rows * in; i += blockDim.x) {
        const int r = i / in, c = i - r * in;
        xs[i] = llb_to_float(x[(size_t)(t0 + r) * x_stride + x_off + (size_t)h * in + c]);
    }
    __syncthreads();
    const T* wh = w + (size_t)h * on * in;
    // a thread owns output column o for all rows of the tile: its weight row is read once
    for (int o = threadIdx.x; o < on; o += blockDim.x) {
        float acc[HL_ROWS];
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.0f;
        const T* wr = wh + (size_t)o * in;
        for (int i = 0; i < in; ++i) {
            const float wv = llb_to_float(wr[i]);
#pragma unroll
            for (int r = 0; r < HL_ROWS; ++r) acc[r] = fmaf(xs[r * in + i], wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r)
            if (r < rows) out[((size_t)(t0 + r) * H + h) * on + o] = llb_from_float<T>(acc[r]);
    }
}

}  // namespace

// x: row t starts at x + t * x_stride + x_off and holds H*in values; w [H, on, in]; out [T, H*on].
LLB_EXPORT int llb_head_linear(const void* x, long long x_stride, int x_off, const void* w, void* out, int dtype, int T,
                               int H, int in, int on, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && H > 0 && in > 0 && on > 0 && x && w && out, "head_linear: bad arguments");
    const size_t smem = (size_t)HL_ROWS * in * sizeof(float);
    LLB_REQUIRE(smem <= 48 * 1024, "head_linear: %d input features per head need %zu bytes of shared memory", in, smem);
    LLB_REQUIRE(H <= 65535, "head_linear: too many heads");
    dim3 grid((T + HL_ROWS - 1) / HL_ROWS, H);
    // zero rows beyond the tile's end are never read: acc of such rows is dropped
    if (dtype == LLB_F32)
        head_linear_kernel<float><<<grid, 256, smem, stream>>>((const float*)x, x_stride, x_off, (const float*)w,
                                                               (float*)out, T, H, in, on);
    else if (dtype == LLB_BF16)
        head_linear_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>((const __nv_bfloat16*)x, x_stride, x_off,
                                                                       (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, H,
                                                                       in, on);
    else
        return llb_fail("head_linear: unknown dtype %d", dtype);
    return llb_check_launch("head_linear");
}
