// Embedding gather: residual[t, :] = table[ids[t], :], written in 32-bit.
//
// Reference op: row gather with an out-of-vocabulary error
// (backends/cpu/src/backend.rs:282-298). Here the host rejects bad ids before
// the launch; a bad id that still reaches the device writes zeros and sets
// kStatusBadToken in the status word.
#include "common.cuh"

namespace {

template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab,
                                 int* __restrict__ status) {
    qi::pdl_enter();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, qi::kStatusBadToken);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = qi::to_f32<TW>(src[i]);
}

}  // namespace

extern "C" int qi_embedding(const void* table, int table_dtype, const int* ids, float* out,
                            int n_tokens, int hidden, int vocab, int* status,
                            cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes n=%d hidden=%d vocab=%d",
               n_tokens, hidden, vocab);
    if (n_tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    QI_DISPATCH_DTYPE(table_dtype, TW, {
        qi::launch(embedding_kernel<TW>, dim3(n_tokens), dim3(threads), 0, stream, (const TW*)table, ids, out, hidden, vocab,
                   status);
    });
    return qi::check_launch("embedding");
}
