// Token embedding gather into the float residual stream.
//
// out[t, :] = table[ids[t], :] * scale  (src/ops/embedding.cu:9-18; the scale is 1 there).  A second destination may keep
// the same rows in float or bf16 for layers that read the embedding again later.  The reference replaces an id
// outside [0, V) by 0; here such an id writes zeros and raises the device error flag, which
// the engine reports as an error.
#include "common.cuh"

template <typename TW, typename TC>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int D, int V, int* __restrict__ err, float scale,
                                 TC* __restrict__ copy) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0 && err) atomicExch(err, 1);
    const TW* row = table + (size_t)(ok ? id : 0) * D;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = ok ? llb_to_float(row[d]) * scale : 0.0f;
        o[d] = v;
        if (copy) copy[(size_t)t * D + d] = llb_from_float<TC>(v);
    }
}

// ids [T] int32, table [V, D] (float or bf16), out [T, D] float, err: one int or null.
LLB_EXPORT int llb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int D,
                             int V, int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && V > 0, "embedding: bad sizes T=%d D=%d V=%d", T, D, V);
    const int threads = D >= 256 ? 256 : 128;
    if (table_dtype == LLB_F32)
        embedding_kernel<float, float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, D, V, err, 1.0f, nullptr);
    else if (table_dtype == LLB_BF16)
        embedding_kernel<__nv_bfloat16, float><<<T, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, D, V, err,
                                                                         1.0f, nullptr);
    else
        return llb_fail("embedding: unknown table dtype %d", table_dtype);
    return llb_check_launch("embedding");
}

// The same with out = table[ids] * scale, and `copy` ([T, D] in the table's dtype, or null) receiving the same rows.
LLB_EXPORT int llb_embedding_scaled(const int* ids, const void* table, int table_dtype, float* out, int T, int D, int V,
                                    int* err, float scale, void* copy, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && V > 0, "embedding: bad sizes T=%d D=%d V=%d", T, D, V);
    const int threads = D >= 256 ? 256 : 128;
    if (table_dtype == LLB_F32)
        embedding_kernel<float, float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, D, V, err, scale, (float*)copy);
    else if (table_dtype == LLB_BF16)
        embedding_kernel<__nv_bfloat16, __nv_bfloat16><<<T, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, D, V,
                                                                                 err, scale, (__nv_bfloat16*)copy);
    else
        return llb_fail("embedding: unknown table dtype %d", table_dtype);
    return llb_check_launch("embedding");
}
