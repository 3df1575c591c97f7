// The two products of routed experts (see experts.cu) on the tensor cores, bfloat16 with float32 sums: a CTA takes one
// tile of 64 listed rows, all of one expert, by 64 output columns, and walks K in steps of 64 with cp.async in two
// stages; four warps of 16 rows each, mma.sync m16n8k16.  The gated product fetches the gate rows and the up rows of its
// columns side by side and stores silu(gate) * up; the rows of the first product are gathered by token, the rows of
// the second are scattered to their (token, choice) pair.  K must be a multiple of 8 (rows on 16-byte boundaries).
#include "common.cuh"
#include "activations.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 64, THREADS = 128;

__device__ __forceinline__ int tile_at(int row, int col) {      // element offset in a [rows][64] tile, 16-byte pieces swizzled
    return row * BK + ((((col >> 3) ^ (row & 7))) << 3) + (col & 7);
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <bool GATED>
__global__ void __launch_bounds__(THREADS) moe_product_mma_kernel(const bf16* __restrict__ x, const int* __restrict__ sorted_rows,
                                                                  const int* __restrict__ tile_expert, const bf16* __restrict__ weight,
                                                                  bf16* __restrict__ out, int n, int k, int top, int block, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int expert = tile_expert[blockIdx.x];
    if (expert < 0) return;
    constexpr int NB = GATED ? 2 : 1;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* a_tiles = reinterpret_cast<bf16*>(smem_raw);          // [2][BM][BK]
    bf16* b_tiles = a_tiles + 2 * BM * BK;                       // [2][NB][BN][BK]
    __shared__ int row_of[BM];
    const int row0 = blockIdx.x * BM, col0 = blockIdx.y * BN;
    if (threadIdx.x < BM) row_of[threadIdx.x] = sorted_rows[row0 + threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* w = weight + (size_t)expert * NB * n * k;

    auto fetch = [&](int stage, int k0) {
        bf16* a = a_tiles + stage * BM * BK;
        for (int idx = threadIdx.x; idx < BM * (BK / 8); idx += THREADS) {
            const int r = idx / (BK / 8), c = idx % (BK / 8);
            const int pair = row_of[r];
            const bool valid = pair >= 0 && k0 + c * 8 < k;
            const bf16* src = valid ? x + (size_t)(GATED ? pair / top : row0 + r) * k + k0 + c * 8 : x;
            cp_async16(a + tile_at(r, c * 8), src, valid);
        }
#pragma unroll
        for (int half = 0; half < NB; ++half) {
            bf16* b = b_tiles + (stage * NB + half) * BN * BK;
            for (int idx = threadIdx.x; idx < BN * (BK / 8); idx += THREADS) {
                const int r = idx / (BK / 8), c = idx % (BK / 8);
                const bool valid = col0 + r < n && k0 + c * 8 < k;
                const int col = col0 + r;
                const int w_row = block ? col / block * 2 * block + col % block + half * block : half * n + col;     // blocks of gate and up rows, or all gate rows first
                const bf16* src = valid ? w + (size_t)w_row * k + k0 + c * 8 : w;
                cp_async16(b + tile_at(r, c * 8), src, valid);
            }
        }
    };

    float acc[NB][BN / 8][4];
#pragma unroll
    for (int half = 0; half < NB; ++half)
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[half][nt][e] = 0.0f;

    const int steps = (k + BK - 1) / BK;
    fetch(0, 0);
    cp_async_commit();
    for (int i = 0; i < steps; ++i) {
        const int stage = i & 1;
        if (i + 1 < steps) fetch(stage ^ 1, (i + 1) * BK);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* a = a_tiles + stage * BM * BK;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t fa[4];
            ldmatrix_x4(fa, a + tile_at(warp * 16 + (lane & 15), kk * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int half = 0; half < NB; ++half) {
                const bf16* b = b_tiles + (stage * NB + half) * BN * BK;
#pragma unroll
                for (int nt = 0; nt < BN / 8; nt += 2) {
                    uint32_t fb[4];
                    ldmatrix_x4(fb, b + tile_at(nt * 8 + (lane & 7) + ((lane >> 4) << 3), kk * 16 + ((lane >> 3) & 1) * 8));
                    mma_bf16(acc[half][nt], fa, fb[0], fb[1]);
                    mma_bf16(acc[half][nt + 1], fa, fb[2], fb[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = warp * 16 + (lane >> 2) + 8 * rr;
        const int pair = row_of[r];
        if (pair < 0) continue;
        bf16* dst = out + (size_t)(GATED || act >= 0 ? row0 + r : pair) * n;
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = col0 + nt * 8 + 2 * (lane & 3) + e;
                if (col >= n) continue;
                float v = acc[0][nt][2 * rr + e];
                if (GATED) {
                    const float g = round_bf16(v), u = round_bf16(acc[NB - 1][nt][2 * rr + e]);     // the projections' own rounding
                    v = g / (1.0f + expf(-g)) * u;
                } else if (act >= 0) {
                    v = mrs_activate(v, act);
                }
                dst[col] = __float2bfloat16_rn(v);
            }
    }
}

template <bool GATED> constexpr size_t smem_bytes() { return (size_t)(2 * BM * BK + 2 * (GATED ? 2 : 1) * BN * BK) * sizeof(bf16); }

}  // namespace

MRS_EXPORT int mrs_moe_mma_tile() { return BM; }

// As mrs_moe_product_simt (`block` and `act` too), bfloat16 only, lists in tiles of mrs_moe_mma_tile() rows, k a multiple of 8.
MRS_EXPORT int mrs_moe_product_mma(int gated, const void* x, const int* sorted_rows, const int* tile_expert, const void* weight, void* out,
                                   int capacity, int n, int k, int top, int block, int act, void* stream) {
    if (capacity <= 0) return 0;
    if (capacity % BM || n <= 0 || k <= 0 || k % 8 || top <= 0 || (((uintptr_t)x | (uintptr_t)weight) & 15) || block < 0 ||
        (block && (!gated || n % block)) || act > 4 || (gated && act >= 0))
        return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(moe_product_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<true>());
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(moe_product_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<false>());
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const dim3 grid(capacity / BM, (n + BN - 1) / BN);
    if (gated)
        MRS_LAUNCH(moe_product_mma_kernel<true>, grid, THREADS, smem_bytes<true>(), stream, (const bf16*)x, sorted_rows, tile_expert,
                   (const bf16*)weight, (bf16*)out, n, k, top, block, act);
    else
        MRS_LAUNCH(moe_product_mma_kernel<false>, grid, THREADS, smem_bytes<false>(), stream, (const bf16*)x, sorted_rows, tile_expert,
                   (const bf16*)weight, (bf16*)out, n, k, top, block, act);
    MRS_RETURN_LAUNCH_STATUS();
}
