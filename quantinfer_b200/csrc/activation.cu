// The gate of a gated feed-forward: out[t, i] = act(gate[t, i]) * up[t, i], where one fused
// projection wrote gate and up into one row of width 2I: either side by side
// (gate_up[t, 0:I] and gate_up[t, I:2I]) or interleaved (gate_up[t, 2i] and
// gate_up[t, 2i + 1]; the layout whose pairs one GEMM epilogue thread holds).
// The activation is a parameter of the feed-forward part:
//   silu       g / (1 + exp(-g)), in the reference's form (division, then the product;
//              backends/cpu/src/backend.rs:224-238, :235): the only one the reference's model uses
//   gelu       g * 0.5 * (1 + erf(g / sqrt 2))
//   gelu_tanh  g * 0.5 * (1 + tanh(sqrt(2 / pi) * (g + 0.044715 g^3)))
//   relu       max(g, 0)
// (the reference's description of a model names Gelu and Relu beside Silu and uses neither,
// crates/quantinfer-model/src/semantic.rs:26-30). All in 32-bit.
#include "common.cuh"

namespace {

enum Act : int { kSilu = 0, kGelu = 1, kGeluTanh = 2, kRelu = 3 };

template <int ACT> __device__ __forceinline__ float act(float g) {
    if (ACT == kSilu) return g / (1.0f + expf(-g));
    if (ACT == kGelu) return g * 0.5f * (1.0f + erff(g * 0.70710678118654752f));
    if (ACT == kGeluTanh) return g * 0.5f * (1.0f + tanhf(0.79788456080286536f * (g + 0.044715f * g * g * g)));
    return fmaxf(g, 0.f);
}

template <typename T, int ACT>
__global__ void act_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_tokens,
                               int inter, int interleaved) {
    qi::pdl_enter();
    const size_t total = (size_t)n_tokens * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter, i = idx % inter;
        const T* row = gate_up + t * 2 * inter;
        const float g = qi::to_f32<T>(interleaved ? row[2 * i] : row[i]);
        const float u = qi::to_f32<T>(interleaved ? row[2 * i + 1] : row[inter + i]);
        out[idx] = qi::from_f32<T>(act<ACT>(g) * u);
    }
}

}  // namespace

// activation: 0 silu, 1 gelu (erf), 2 gelu_tanh, 3 relu.
extern "C" int qi_act_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter, int interleaved,
                          int activation, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && inter > 0, "act_mul: bad sizes n=%d inter=%d", n_tokens, inter);
    QI_REQUIRE(activation >= 0 && activation <= 3, "act_mul: unknown activation code %d", activation);
    if (n_tokens == 0) return 0;
    const size_t total = (size_t)n_tokens * inter;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    QI_DISPATCH_DTYPE(dtype, T, {
        const T* in = (const T*)gate_up;
        T* o = (T*)out;
        const dim3 grid((unsigned)blocks), block(256);
        switch (activation) {
            case kSilu: qi::launch(act_mul_kernel<T, kSilu>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            case kGelu: qi::launch(act_mul_kernel<T, kGelu>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            case kGeluTanh: qi::launch(act_mul_kernel<T, kGeluTanh>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            default: qi::launch(act_mul_kernel<T, kRelu>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
        }
    });
    return qi::check_launch("act_mul");
}

extern "C" int qi_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter,
                           int interleaved, cudaStream_t stream) {
    return qi_act_mul(gate_up, out, dtype, n_tokens, inter, interleaved, 0, stream);
}
