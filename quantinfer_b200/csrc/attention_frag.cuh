// Fragment-level pieces shared by the attention kernels: ldmatrix / mma.sync wrappers,
// the online softmax step, and the two matrix products of a key tile, written against an
// `Addr` type that maps (row, 16-byte chunk) of a shared-memory tile to a byte offset, so
// that the same code serves tiles filled by cp.async (one swizzled row per key) and tiles
// filled by TMA (64-column halves with the 128-byte swizzle).
#pragma once

#include "common.cuh"

#include <math.h>

namespace qi_attn {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (about 2 ulp), for score differences <= 0.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Rows of D bf16, the 16-byte chunk index XORed with the row's low three bits.
template <int D> struct RowSwizzle {
    static __device__ __forceinline__ uint32_t off(int row, int chunk) {
        return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
    }
};
// What TMA writes with the 128-byte swizzle for boxes of 64 columns: the tile is stored as
// D / 64 halves of ROWS rows of 128 bytes; the tile's base is 1024-byte aligned.
template <int ROWS> struct TmaSwizzle {
    static __device__ __forceinline__ uint32_t off(int row, int chunk) {
        return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
    }
};

// The query fragments (A operand) of 16 rows starting at `row0`.
template <int D, typename Addr>
__device__ __forceinline__ void load_q_frags(uint32_t (&qa)[D / 16][4], uint32_t q_smem, int row0, int lane) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int row = row0 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(q_smem + Addr::off(row, ks * 2 + (lane >> 4)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    }
}

// One warp: scores of its 16 query rows against NT * 8 keys starting at tile row `krow0`.
template <int D, int NT, typename Addr>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const uint32_t (&qa)[D / 16][4], uint32_t k_smem, int krow0, int lane) {
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
            uint32_t r0, r1, r2, r3;
            const int row = krow0 + jp * 16 + (lane & 7) + (lane >> 4) * 8;
            const int chunk = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(k_smem + Addr::off(row, chunk), r0, r1, r2, r3);
            mma_bf16(s[2 * jp], qa[ks], r0, r1);
            mma_bf16(s[2 * jp + 1], qa[ks], r2, r3);
        }
    }
}

// One warp: o += p . v for its 16 rows and NT * 8 keys starting at tile row `krow0`.
template <int D, int NT, typename Addr>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&p)[NT][4], uint32_t v_smem, int krow0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
        pa[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
        pa[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
        pa[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
        for (int nd = 0; nd < D / 16; ++nd) {
            uint32_t r0, r1, r2, r3;
            const int row = krow0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int chunk = nd * 2 + (lane >> 4);
            ldmatrix_x4_trans(v_smem + Addr::off(row, chunk), r0, r1, r2, r3);
            mma_bf16(o[2 * nd], pa, r0, r1);
            mma_bf16(o[2 * nd + 1], pa, r2, r3);
        }
    }
}

// Online softmax over one tile of raw scores (masked entries are -inf): with
// c = scale * log2 e, updates the running maximum m (of c * score) and the sum l of the
// two rows this thread holds (g and g + 8), rescales o, and leaves the weights
// 2^(c * score - m) in s.
template <int D, int NT>
__device__ __forceinline__ void softmax_tile(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4], float c) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], ms[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float mn = fmaxf(m[r], mx[r] * c);           // c > 0; -inf stays -inf
        ms[r] = (mn == -INFINITY) ? 0.f : mn;               // a row with no key yet: every weight is 2^-inf = 0
        corr[r] = ex2(m[r] - ms[r]);                        // m = -inf gives 0
        m[r] = mn;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const float p = ex2(fmaf(s[j][e], c, -ms[r]));
            s[j][e] = p;
            sum[r] += p;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + sum[r];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
    }
}

}  // namespace qi_attn
