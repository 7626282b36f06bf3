// Plain matrix product on the 32-bit FMA pipe: y[M, N] = x[M, K] . w[N, K]^T.
//
// `w` is in the checkpoint's [out, in] layout, so both operands are read along
// K. Any element type for x, w and y; products and sums are 32-bit, and every
// output element is accumulated by one thread with k ascending, so a row's
// result does not depend on which other rows are in the batch. This is the
// matrix product of the true 32-bit path (no tensor cores, no TF32) and of
// any operand combination the tensor-core kernel does not take. The reference
// computes out[c] = sum_k x[k] * W[k, c] with k ascending
// (backends/cpu/src/matmul.rs:50-59).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int M,
                 int N, int K, long long ldx, long long ldw, long long ldy) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    qi::pdl_enter();
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // tx over N, ty over M
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // Each thread loads 4 consecutive k of one row of each tile.
    const int lrow = tid / 4;        // 0..63
    const int lk = (tid % 4) * 4;    // 0,4,8,12
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            float a = 0.f, b = 0.f;
            if (k < K) {
                if (m0 + lrow < M) a = qi::to_f32<TX>(x[(size_t)(m0 + lrow) * ldx + k]);
                if (n0 + lrow < N) b = qi::to_f32<TW>(w[(size_t)(n0 + lrow) * ldw + k]);
            }
            xs[lk + i][lrow] = a;
            ws[lk + i][lrow] = b;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) y[(size_t)m * ldy + n] = qi::from_f32<TY>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TY>
int launch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx,
           long long ldw, long long ldy, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    qi::launch(gemm_simt_kernel<TX, TW, TY>, grid, dim3(256), 0, stream, (const TX*)x, (const TW*)w, (TY*)y, M, N, K, ldx, ldw,
               ldy);
    return qi::check_launch("gemm_simt");
}

}  // namespace

extern "C" int qi_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y,
                            int y_dtype, int M, int N, int K, long long ldx, long long ldw,
                            long long ldy, cudaStream_t stream) {
    QI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    QI_REQUIRE(ldx >= K && ldw >= K && ldy >= N, "gemm_simt: a leading dimension is smaller than its row");
    QI_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_simt: M=%d is too large for one launch", M);
    if (M == 0) return 0;
    QI_DISPATCH_DTYPE(x_dtype, TX, {
        QI_DISPATCH_DTYPE(w_dtype, TW, {
            QI_DISPATCH_DTYPE(y_dtype, TY, {
                return launch<TX, TW, TY>(x, w, y, M, N, K, ldx, ldw, ldy, stream);
            });
        });
    });
    return 0;
}
