// A decode step's traffic with the host, done by two tiny kernels instead of copy-engine
// transfers, so that nothing between two steps leaves the compute queue.
//
// stage_step: the step's packed batch arrays (positions, lengths, block tables ...) are read
// straight from the pinned host buffer they were packed into (pinned memory is addressable
// from the device) and written to the device buffer the step's kernels read; the token ids
// at its front come from the device (the tokens the step before sampled) when given.
//
// publish: the status word and the sampled tokens are written to a pinned host buffer, which
// the host reads after the event that follows this kernel.
//
// The reference copies inputs and results with the runtime's transfer calls
// (backends/cuda/src/native.rs:100-126: clone_htod of the operands, clone_dtoh of the result); here the bytes
// are the same and only the engine that moves them differs.
#include "common.cuh"

namespace {

// This kernel does not release its successor early (no launch_dependents): the kernels of the
// step read lengths and block tables before their own wait for their predecessor, which is only
// safe once these arrays are complete, so the step's first kernel starts when this one has ended.
__global__ void stage_step_kernel(const int* __restrict__ host_meta, int* __restrict__ meta, int n,
                                  const int* __restrict__ device_tokens, int n_tokens) {
    qi::pdl_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        meta[i] = (device_tokens && i < n_tokens) ? device_tokens[i] : host_meta[i];
}

__global__ void publish_kernel(const int* __restrict__ src, int* __restrict__ host_out, int n) {
    qi::pdl_enter();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) host_out[i] = src[i];
    __threadfence_system();
}

}  // namespace

// meta[0, n) = host_meta[0, n), except meta[0, n_tokens) = device_tokens when that is not null.
// host_meta must be pinned host memory (its address is used on the device).
extern "C" int qi_stage_step(const int* host_meta, int* meta, int n, const int* device_tokens, int n_tokens,
                             cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && n_tokens >= 0 && n_tokens <= n, "stage_step: bad sizes n=%d tokens=%d", n, n_tokens);
    if (n == 0) return 0;
    const int blocks = (n + 255) / 256 < 32 ? (n + 255) / 256 : 32;
    qi::launch(stage_step_kernel, dim3(blocks), dim3(256), 0, stream, host_meta, meta, n, device_tokens, n_tokens);
    return qi::check_launch("stage_step");
}

// host_out[0, n) = src[0, n); host_out must be pinned host memory.
extern "C" int qi_publish(const int* src, int* host_out, int n, cudaStream_t stream) {
    QI_REQUIRE(n >= 0, "publish: bad size %d", n);
    if (n == 0) return 0;
    const int blocks = (n + 255) / 256 < 8 ? (n + 255) / 256 : 8;
    qi::launch(publish_kernel, dim3(blocks), dim3(256), 0, stream, src, host_out, n);
    return qi::check_launch("publish");
}
