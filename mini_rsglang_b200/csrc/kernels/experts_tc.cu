// The two products of routed experts (see experts.cu) for many rows (prompt portions) on the tcgen05 tensor cores,
// bfloat16 in, float32 accumulation.  The listed rows are first gathered expert by expert into one matrix
// (mrs_moe_gather_rows in experts.cu), so that a tile of 128 rows, all of one expert, comes in by bulk tensor copies;
// the experts' weights are one matrix [experts * rows an expert, K], and a tile's weight rows start at its expert's
// first row.  As in gemm_many_rows.cu a CTA computes a tile of 128 rows x 256 weight rows into one of two
// accumulators in tensor memory while four warps turn the other, finished one into values:
//   warp 0   fetches 128 x 64 row tiles and 256 x 64 weight tiles (TMA, 128-byte swizzle) into a ring of stages;
//   warp 1   one thread issues tcgen05.mma (M 128, N 256, K 16) on the stages;
//   warps 2-5 a thread a row: the row's 256 sums from tensor memory;
//             gated: a weight tile holds two blocks of 64 gate and 64 up rows, out[row] = silu(gate) * up;
//             plain: out[pair of the row] = the sums (the rows go back to their (token, choice) pairs).
// Only the tiles that the lists use are walked: their count stands behind the tiles' experts.  CTAs are
// persistent; tiles that share a weight tile are taken by neighbouring CTAs at the same time.  Every wait is bounded
// (tma.cuh).
#include "tcgen05.cuh"
#include "activations.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4, THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLUMNS = 2 * BN;
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 16;

// x_map: the gathered rows [capacity, K]; w_map: the weights [experts * N, K]; N: weight rows an expert.
// tile_expert [capacity / 128 + 1]: the expert of every tile of rows, then the number of tiles in use.
template <bool GATED>
__global__ void __launch_bounds__(THREADS, 1) moe_product_tc_kernel(
    const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, const int* __restrict__ tile_expert,
    const int* __restrict__ sorted_rows, bf16* __restrict__ out, int m_tiles_all, int N, int K, int act) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BK - 1) / BK;
    const int n_tiles = (N + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLUMNS);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();
    int m_tiles = tile_expert[m_tiles_all];                   // tiles of rows in use (the lists are packed from the front)
    m_tiles = m_tiles < 0 ? 0 : (m_tiles > m_tiles_all ? m_tiles_all : m_tiles);
    const int tiles = m_tiles * n_tiles;                      // tile t: weight tile t / m_tiles, row tile t % m_tiles

    if (warp == 0) {
        const bool leader = elect_one();
        if (leader) {
            tma_prefetch_descriptor(&x_map);
            tma_prefetch_descriptor(&w_map);
        }
        int it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int m_tile = tile % m_tiles;
            const int expert = max(tile_expert[m_tile], 0);
            const int m0 = m_tile * BM, n0 = expert * N + (tile / m_tiles) * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (!(alive = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1))) break;
                unsigned char* stage = smem + s * STAGE_BYTES;
                if (leader) {
                    mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(stage, &x_map, &full[s], kb * BK, m0);
                    tma_load_2d(stage + A_BYTES, &w_map, &full[s], kb * BK, n0);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        const bool leader = elect_one();
        constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BN);
        int it = 0, round = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++round) {
            const int buffer = round & 1;
            if (!(alive = mbar_wait(&acc_empty[buffer], ((round >> 1) & 1) ^ 1))) break;
            tcgen05_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buffer * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (!(alive = mbar_wait(&full[s], (it / STAGES) & 1))) break;
                tcgen05_fence_after_sync();
                const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(smem + s * STAGE_BYTES));
                const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(smem + s * STAGE_BYTES + A_BYTES));
                if (leader) {
                    if (kb > 0) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_more(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc);
                    } else {
                        umma_bf16_first(d_tmem, a_desc, b_desc, idesc);
#pragma unroll
                        for (int k = 1; k < BK / UMMA_K; ++k) umma_bf16_more(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc);
                    }
                    umma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (leader) umma_commit(&acc_full[buffer]);
            __syncwarp();
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // row within the tile
        int round = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++round) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const int buffer = round & 1;
            mbar_wait(&acc_full[buffer], (round >> 1) & 1);
            __syncwarp();
            tcgen05_fence_after_sync();
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buffer * BN;
            const int pair = sorted_rows[m0 + row];
            if (GATED) {
                const int half_n = N >> 1;
                bf16* dst = out + (size_t)(m0 + row) * half_n + (n0 >> 1);
#pragma unroll
                for (int block = 0; block < BN / 128; ++block) {          // 64 gate columns, then their 64 up columns
#pragma unroll
                    for (int c = 0; c < 64; c += 32) {
                        float g[32], u[32];
                        tmem_load_32_async(acc + block * 128 + c, g);
                        tmem_load_32_async(acc + block * 128 + 64 + c, u);
                        tmem_load_wait();
                        if (pair >= 0 && n0 + block * 128 < N) {
#pragma unroll
                            for (int e = 0; e < 32; e += 8) {
                                uint32_t w[4];
#pragma unroll
                                for (int p = 0; p < 4; ++p) {
                                    const float g0 = __bfloat162float(__float2bfloat16_rn(g[e + 2 * p])), g1 = __bfloat162float(__float2bfloat16_rn(g[e + 2 * p + 1]));
                                    const float u0 = __bfloat162float(__float2bfloat16_rn(u[e + 2 * p])), u1 = __bfloat162float(__float2bfloat16_rn(u[e + 2 * p + 1]));
                                    __nv_bfloat162 two = __floats2bfloat162_rn(g0 / (1.0f + __expf(-g0)) * u0, g1 / (1.0f + __expf(-g1)) * u1);
                                    w[p] = *reinterpret_cast<uint32_t*>(&two);
                                }
                                *reinterpret_cast<uint4*>(dst + block * 64 + c + e) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            } else {
                bf16* dst = out + (size_t)(pair < 0 ? 0 : (act >= 0 ? m0 + row : pair)) * N + n0;
#pragma unroll
                for (int c = 0; c < BN; c += 32) {
                    float v[32];
                    tmem_load_32_async(acc + c, v);
                    tmem_load_wait();
                    if (pair >= 0) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            if (n0 + c + e + 8 > N) continue;           // N is a multiple of 8
                            uint32_t w[4];
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                __nv_bfloat162 two = act >= 0 ? __floats2bfloat162_rn(mrs_activate(v[e + 2 * p], act), mrs_activate(v[e + 2 * p + 1], act))
                                                              : __floats2bfloat162_rn(v[e + 2 * p], v[e + 2 * p + 1]);
                                w[p] = *reinterpret_cast<uint32_t*>(&two);
                            }
                            *reinterpret_cast<uint4*>(dst + c + e) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buffer]);
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

}  // namespace

MRS_EXPORT int mrs_moe_tc_tile() { return BM; }

// A tensor map of a row-major bfloat16 matrix [rows, cols] for copies of `box_rows` rows x 64 columns
// (128 rows for the gathered rows, 256 for the weights).
MRS_EXPORT int mrs_moe_tc_map(const void* base, long long rows, long long cols, int box_rows, void* map_out) {
    if (rows <= 0 || cols <= 0 || cols % 8 || box_rows <= 0 || box_rows > 256 || ((uintptr_t)base & 15)) return MRS_BAD_ARGUMENT;
    const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
    const uint64_t strides[1] = {(uint64_t)cols * 2};
    const uint32_t box[2] = {BK, (uint32_t)box_rows};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// gated != 0: x_map over the gathered rows [capacity, K], w_map over [experts * N, K] with, in every block of 128 rows,
// 64 gate rows and then the 64 matching up rows (N a multiple of 128), out [capacity, N / 2] = silu(gate) * up.
// Else: x_map over [capacity, K], w_map over [experts * N, K] (N a multiple of 8), out [pairs, N] written at the rows'
// pairs; or, with act >= 0 (an activation's number), out [capacity, N] = activation of the sums, at the rows' places.
// tile_expert [capacity / 128 + 1] as mrs_moe_align leaves it for tiles of 128 rows; `ctas`: the GPU's SMs.
MRS_EXPORT int mrs_moe_product_tc(int gated, const void* x_map, const void* w_map, const int* tile_expert, const int* sorted_rows,
                                  void* out, int capacity, int N, int K, int act, int ctas, void* stream) {
    if (capacity <= 0) return 0;
    if (capacity % BM || K <= 0 || K % 8 || N <= 0 || (gated ? N % 128 : N % 8) || ctas < 1 || !x_map || !w_map || !out ||
        ((uintptr_t)out & 15) || act > 4 || (gated && act >= 0))
        return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(moe_product_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_product_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = capacity / BM;
    const long long tiles = (long long)m_tiles * ((N + BN - 1) / BN);
    const int grid = (int)(ctas < tiles ? ctas : tiles);
    if (gated)
        MRS_LAUNCH(moe_product_tc_kernel<true>, grid, THREADS, SMEM_BYTES, stream, *reinterpret_cast<const CUtensorMap*>(x_map),
                   *reinterpret_cast<const CUtensorMap*>(w_map), tile_expert, sorted_rows, (bf16*)out, m_tiles, N, K, act);
    else
        MRS_LAUNCH(moe_product_tc_kernel<false>, grid, THREADS, SMEM_BYTES, stream, *reinterpret_cast<const CUtensorMap*>(x_map),
                   *reinterpret_cast<const CUtensorMap*>(w_map), tile_expert, sorted_rows, (bf16*)out, m_tiles, N, K, act);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_moe_tc_take_error(unsigned int* word) { return mrs_take_error_word(word); }
MRS_EXPORT int mrs_moe_tc_mirror_errors(unsigned int* host_word) { return mrs_set_error_mirror(host_word); }

MRS_EXPORT const char* mrs_moe_tc_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (K or N no multiple of 8, gated N no multiple of 128, unaligned base)";
    if (code == MRS_TENSOR_MAP_FAILED) return "the driver refused the tensor map (address, sizes or strides)";
    return cudaGetErrorString((cudaError_t)code);
}
