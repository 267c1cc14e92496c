// SwiGLU gate:  out[t,j] = silu(g) * u with g = gu[t,2j], u = gu[t,2j+1], silu(g) = g / (1 + expf(-g))
// (formula of src/operators/cuda/cuda_elementwise.cu:34-41).  The gate and up projections are stored
// with their rows interleaved, so one GEMM yields [T, 2I] with each (gate, up) pair adjacent.
// act 1: the gate's activation is gelu_tanh(g) = g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) instead.
#include "common.cuh"

namespace {

template <typename TOut>
__global__ void silu_mul_interleaved_kernel(const float* __restrict__ gu, TOut* __restrict__ out, size_t n, int act) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float2 p = reinterpret_cast<const float2*>(gu)[i];
    const float g = act == 1 ? 0.5f * p.x * (1.0f + tanhf(0.7978845608028654f * (p.x + 0.044715f * p.x * p.x * p.x)))
                             : p.x / (1.0f + expf(-p.x));
    out[i] = forge::from_float<TOut>(g * p.y);
}

// out[t][c] = act(in[t * ld + c]) in the output type, for the first n columns of fp32 rows: the activation between the two
// products of an ungated feed-forward.  act 0: the exact gelu, z/2 (1 + erf(z / sqrt 2)); 1: its tanh form; 2: silu.
template <typename TOut>
__global__ void act_rows_kernel(const float* __restrict__ in, int ld, TOut* __restrict__ out, size_t total, int n, int act) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float z = in[(i / n) * ld + i % n];
    float y;
    if (act == 0) y = 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
    else if (act == 1) y = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    else y = z / (1.0f + expf(-z));
    out[i] = forge::from_float<TOut>(y);
}

}  // namespace

extern "C" int forge_act_rows(const float* in, int ld, void* out, int out_dtype, int T, int n, int act, cudaStream_t stream) {
    if (T < 0 || n <= 0 || ld < n || act < 0 || act > 2) return forge::fail(FORGE_ERR_ARG, "act_rows: bad sizes T=%d n=%d ld=%d act=%d", T, n, ld, act);
    const size_t total = (size_t)T * n;
    if (total == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(act_rows_kernel<TO>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1, in, ld, (TO*)out, total, n, act));
    return forge::check_launch("act_rows", e);
}

extern "C" int forge_silu_mul_interleaved(const float* gu, void* out, int out_dtype, int T, int I, int act,
                                          cudaStream_t stream) {
    if (T < 0 || I <= 0) return forge::fail(FORGE_ERR_ARG, "silu_mul: bad sizes T=%d I=%d", T, I);
    const size_t n = (size_t)T * I;
    if (n == 0) return FORGE_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(silu_mul_interleaved_kernel<TO>, dim3(blocks), dim3(256), 0, stream, 1, gu, (TO*)out, n, act));
    return forge::check_launch("silu_mul_interleaved", e);
}
