// Token embedding gather: out[t,:] = table[ids[t],:] * scale, written to the fp32 residual stream (or, with `add`, added to
// it: a design that feeds the embedding into the stream again before a repeated pass of its layers).
// Replaces the reference's embedding_kernel (src/operators/cuda/cuda_embedding.cu:9-34); like it,
// an id outside [0,V) gives a row of zeros, and here it also raises bit 0 of *status.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V, float scale, int add, int* status) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (!add) for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        return;
    }
    const T* row = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = (add ? o[c] : 0.f) + forge::to_float(row[c]) * scale;
}

}  // namespace

extern "C" int forge_embedding(const int32_t* ids, const void* table, int table_dtype, float* out,
                               int T, int H, int V, float scale, int add, int* status, cudaStream_t stream) {
    if (T < 0 || H <= 0 || V <= 0) return forge::fail(FORGE_ERR_ARG, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return FORGE_OK;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(table_dtype, TT,
        e = forge::launch(embedding_kernel<TT>, dim3(T), dim3(threads), 0, stream, 1, ids, (const TT*)table, out, H, V, scale, add, status));
    return forge::check_launch("embedding", e);
}
