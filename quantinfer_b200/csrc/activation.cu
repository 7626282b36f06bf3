// SwiGLU gate: out[t, i] = silu(gate[t, i]) * up[t, i], where one fused
// projection wrote gate and up into one row of width 2I: either side by side
// (gate_up[t, 0:I] and gate_up[t, I:2I]) or interleaved (gate_up[t, 2i] and
// gate_up[t, 2i + 1]; the layout whose pairs one GEMM epilogue thread holds).
// silu(g) = g / (1 + exp(-g)), evaluated in 32-bit in the reference's form
// (division, then the product; backends/cpu/src/backend.rs:224-238, :235).
#include "common.cuh"

namespace {

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_tokens,
                                int inter, int interleaved) {
    qi::pdl_enter();
    const size_t total = (size_t)n_tokens * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter, i = idx % inter;
        const T* row = gate_up + t * 2 * inter;
        const float g = qi::to_f32<T>(interleaved ? row[2 * i] : row[i]);
        const float u = qi::to_f32<T>(interleaved ? row[2 * i + 1] : row[inter + i]);
        out[idx] = qi::from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

}  // namespace

extern "C" int qi_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter,
                           int interleaved, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && inter > 0, "silu_mul: bad sizes n=%d inter=%d", n_tokens, inter);
    if (n_tokens == 0) return 0;
    const size_t total = (size_t)n_tokens * inter;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(silu_mul_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (const T*)gate_up, (T*)out, n_tokens, inter,
                   interleaved);
    });
    return qi::check_launch("silu_mul");
}
