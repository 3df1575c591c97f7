// Routed experts with shapes that do not depend on the routing, so that a step can be recorded and replayed:
//
//   moe_route      float32 router logits [tokens, all experts (+ 1 gate of the shared expert)] -> scores by softmax
//                  (or sigmoid) over all experts, the `top` largest of score + correction (ties: the lower number),
//                  their weights score / (sum of the chosen scores + 1e-20) * scale (or, not normalised, score * scale),
//                  sigmoid of the shared gate
//   moe_align      the (token, choice) pairs that go to a routed expert, listed expert by expert, every expert's run
//                  filled up to whole tiles of `tile` rows (-1), the expert of every tile (-1: unused) and, behind
//                  them, the number of tiles in use (the runs are packed from the front);
//                  experts numbered from `routed` on have no weights (they hand their input on) and get no rows
//   moe_gather_rows  the listed pairs' input rows, in the order of the lists (zeros where a run is filled up), each times
//                  its pair's weight if weights are given: the matrix that the product for many rows reads with bulk
//                  tensor copies, and the input of experts whose weight multiplies what they read
//   moe_up / moe_down   the two products of the gated unit over those tiles, on the CUDA cores in float32 sums:
//                  act[row] = silu(W_gate[e] x) * (W_up[e] x),  y[pair] = W_down[e] act[row]; for experts without a gate
//                  the first product is the ungated one over gathered rows with an activation on its sums, written at the
//                  rows' places in the lists (`act` >= 0): act[row] = activation(W_up[e] x_rows[row]);
//                  one kernel for every size (the 32-bit path), one for few rows an expert (decode steps: the
//                  weights streamed once); the tensor-core versions are experts_mma.cu and experts_tc.cu
//   moe_combine    out[token] = sum over its choices of weight * (y[pair] or, for an expert without weights, the
//                  input itself) + shared gate * shared expert's output
//
// A row's result depends on its own pair alone: which other rows share its tile, and the order of a run, do not enter.
#include "common.cuh"
#include "activations.cuh"

namespace {

// One warp a token.  Dynamic shared memory: warps * 2 * all floats (scores, choice scores).
__global__ void moe_route_kernel(const float* __restrict__ logits, int stride, const float* __restrict__ correction,
                                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_gate, int tokens,
                                 int all, int top, float scale, int sigmoid_scores, int has_shared, int normalize) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x * warps + warp;
    if (t >= tokens) return;
    float* score = route_smem + (size_t)warp * 2 * all;
    float* choice = score + all;
    const float* z = logits + (size_t)t * stride;
    float top_z = -CUDART_INF_F;
    for (int e = lane; e < all; e += 32) top_z = fmaxf(top_z, z[e]);
    top_z = warp_max(top_z);
    float sum = 0.0f;
    for (int e = lane; e < all; e += 32) {
        const float s = sigmoid_scores ? 1.0f / (1.0f + expf(-z[e])) : expf(z[e] - top_z);
        score[e] = s;
        sum += s;
    }
    sum = warp_sum(sum);
    const float inv = sigmoid_scores ? 1.0f : 1.0f / sum;
    for (int e = lane; e < all; e += 32) {
        score[e] *= inv;
        choice[e] = score[e] + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    float picked_sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -CUDART_INF_F;
        int best_e = 0x7fffffff;
        for (int e = lane; e < all; e += 32)
            if (choice[e] > best) best = choice[e], best_e = e;       // strided upward: the lower number wins a tie in a lane
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, o);
            const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (other > best || (other == best && other_e < best_e)) best = other, best_e = other_e;
        }
        if (best_e >= all) best_e = 0;          // fewer finite scores than choices: cannot happen with finite logits
        const float s = score[best_e];
        picked_sum += s;
        if (lane == 0) {
            chosen[(size_t)t * top + k] = best_e;
            weights[(size_t)t * top + k] = s;
            choice[best_e] = -CUDART_INF_F;
        }
        __syncwarp();
    }
    const float factor = normalize ? scale / (picked_sum + 1e-20f) : scale;          // not normalised: the scores themselves
    if (normalize) {
        if (lane < top) weights[(size_t)t * top + lane] = weights[(size_t)t * top + lane] / (picked_sum + 1e-20f) * scale;
        for (int k = 32 + lane; k < top; k += 32) weights[(size_t)t * top + k] = weights[(size_t)t * top + k] / (picked_sum + 1e-20f) * scale;
    } else if (scale != 1.0f) {
        for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= factor;
    }
    if (has_shared && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-z[all]));
}

// One block.  Dynamic shared memory: 3 * routed ints (count, first row, filled).
__global__ void moe_align_kernel(const int* __restrict__ chosen, int pairs, int routed, int tile, int* __restrict__ sorted_rows,
                                 int* __restrict__ tile_expert, int capacity) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int align_smem[];
    int* count = align_smem;
    int* first = count + routed;
    int* filled = first + routed;
    for (int e = threadIdx.x; e < routed; e += blockDim.x) count[e] = 0, filled[e] = 0;
    for (int i = threadIdx.x; i < capacity; i += blockDim.x) sorted_rows[i] = -1;
    for (int i = threadIdx.x; i < capacity / tile; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < routed) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < routed; ++e) {
            first[e] = at;
            at += (count[e] + tile - 1) / tile * tile;
        }
        tile_expert[capacity / tile] = at / tile;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < routed; e += blockDim.x)
        for (int i = first[e] / tile; i < (first[e] + count[e] + tile - 1) / tile; ++i) tile_expert[i] = e;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < routed) sorted_rows[first[e] + atomicAdd(&filled[e], 1)] = i;
    }
}

constexpr int SIMT_TM = 32, SIMT_TN = 64, SIMT_TK = 32;

// A tile of 32 rows by 64 output columns of one expert, 256 threads, each 2 rows x 4 columns.
// GATED: the weights hold 2 * n rows an expert (all gate rows, then all up rows; or, with `block`, blocks of `block` gate
// rows each followed by the matching up rows), out[row] = silu(gate) * up, the input row of a listed pair is
// x[pair / top]; else the input row is x[its place in the list] and out is written at the pair.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_product_simt_kernel(const T* __restrict__ x, const int* __restrict__ sorted_rows,
                                                               const int* __restrict__ tile_expert, const T* __restrict__ weight,
                                                               T* __restrict__ out, int n, int k, int top, int block, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int expert = tile_expert[blockIdx.x];
    if (expert < 0) return;
    __shared__ float a_s[SIMT_TM][SIMT_TK + 1];
    __shared__ float b_s[GATED ? 2 : 1][SIMT_TN][SIMT_TK + 1];
    __shared__ int row_of[SIMT_TM];
    const int row0 = blockIdx.x * SIMT_TM, col0 = blockIdx.y * SIMT_TN;
    if (threadIdx.x < SIMT_TM) row_of[threadIdx.x] = sorted_rows[row0 + threadIdx.x];
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* w = weight + (size_t)expert * (GATED ? 2 : 1) * n * k;
    float acc[GATED ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < k; k0 += SIMT_TK) {
        for (int idx = threadIdx.x; idx < SIMT_TM * SIMT_TK; idx += 256) {
            const int r = idx / SIMT_TK, c = idx % SIMT_TK;
            const int pair = row_of[r];
            float v = 0.0f;
            if (pair >= 0 && k0 + c < k) v = to_float(x[(size_t)(GATED ? pair / top : row0 + r) * k + k0 + c]);
            a_s[r][c] = v;
        }
        for (int idx = threadIdx.x; idx < SIMT_TN * SIMT_TK; idx += 256) {
            const int r = idx / SIMT_TK, c = idx % SIMT_TK;
            const bool in = col0 + r < n && k0 + c < k;
            const int col = col0 + r;
            const int gate_row = GATED && block ? col / block * 2 * block + col % block : col;
            b_s[0][r][c] = in ? to_float(w[(size_t)gate_row * k + k0 + c]) : 0.0f;
            if (GATED) b_s[1][r][c] = in ? to_float(w[(size_t)(gate_row + (block ? block : n)) * k + k0 + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < SIMT_TK; ++c) {
            const float a0 = a_s[ty][c], a1 = a_s[ty + 16][c];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = b_s[0][tx + 16 * j][c];
                acc[0][0][j] += a0 * b;
                acc[0][1][j] += a1 * b;
                if (GATED) {
                    const float u = b_s[1][tx + 16 * j][c];
                    acc[1][0][j] += a0 * u;
                    acc[1][1][j] += a1 * u;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty + 16 * i;
        const int pair = row_of[r];
        if (pair < 0) continue;
        T* dst = out + (size_t)(GATED || act >= 0 ? row0 + r : pair) * n;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col0 + tx + 16 * j;
            if (col >= n) continue;
            float v = acc[0][i][j];
            if (GATED) {
                const float g = to_float(from_float<T>(v)), u = to_float(from_float<T>(acc[1][i][j]));   // the projections' own rounding
                v = g / (1.0f + expf(-g)) * u;
            } else if (act >= 0) {
                v = mrs_activate(v, act);
            }
            dst[col] = from_float<T>(v);
        }
    }
}

// Few rows an expert (decode steps): a tile of 4 listed rows by 32 output columns, 8 warps, each 4 columns.  The weights
// are read once, sixteen bytes a lane and step, straight from memory (no staging: nothing is used twice), eight such
// loads in flight a lane; the rows wait in shared memory, 2,048 columns at a time.  The kernel is bound by the weights'
// bytes, which is what a decode step has to move.  k a multiple of 16 bytes.
constexpr int ROWS_TM = 4, ROWS_WARPS = 8, ROWS_J = 4, ROWS_KC = 2048;
template <typename T> struct Piece;            // sixteen bytes of T as floats
template <> struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x, v[1] = r.y, v[2] = r.z, v[3] = r.w;
    }
};
template <> struct Piece<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
    }
};

template <typename T, bool GATED>
__global__ void __launch_bounds__(32 * ROWS_WARPS) moe_product_rows_kernel(const T* __restrict__ x, const int* __restrict__ sorted_rows,
                                                                            const int* __restrict__ tile_expert, const T* __restrict__ weight,
                                                                            T* __restrict__ out, int n, int k, int top, int block, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int expert = tile_expert[blockIdx.x];
    if (expert < 0) return;
    constexpr int V = Piece<T>::N, NB = GATED ? 2 : 1;
    __shared__ __align__(16) T x_s[ROWS_TM][ROWS_KC];
    __shared__ int row_of[ROWS_TM];
    const int row0 = blockIdx.x * ROWS_TM;
    if (threadIdx.x < ROWS_TM) row_of[threadIdx.x] = sorted_rows[row0 + threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* w = weight + (size_t)expert * NB * n * k;
    const int col_base = blockIdx.y * (ROWS_WARPS * ROWS_J);
    const T* w_row[ROWS_J][NB];
#pragma unroll
    for (int j = 0; j < ROWS_J; ++j) {
        const int col = min(col_base + warp + ROWS_WARPS * j, n - 1);          // a column beyond the last repeats it and is not stored
        const int gate_row = GATED && block ? col / block * 2 * block + col % block : col;
        w_row[j][0] = w + (size_t)gate_row * k;
        if (GATED) w_row[j][NB - 1] = w + (size_t)(gate_row + (block ? block : n)) * k;
    }
    float acc[ROWS_J][NB][ROWS_TM] = {};
    for (int kc = 0; kc < k; kc += ROWS_KC) {
        const int len = min(ROWS_KC, k - kc);
        __syncthreads();
        for (int idx = threadIdx.x; idx < ROWS_TM * (len / V); idx += 32 * ROWS_WARPS) {
            const int r = idx / (len / V), c = idx % (len / V);
            const int pair = row_of[r];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (pair >= 0) v = *reinterpret_cast<const uint4*>(x + (size_t)(GATED ? pair / top : row0 + r) * k + kc + c * V);
            *reinterpret_cast<uint4*>(&x_s[r][c * V]) = v;
        }
        __syncthreads();
        for (int i = lane * V; i < len; i += 32 * V) {
            float wv[ROWS_J][NB][V];
#pragma unroll
            for (int j = 0; j < ROWS_J; ++j)
#pragma unroll
                for (int b = 0; b < NB; ++b) Piece<T>::load(w_row[j][b] + kc + i, wv[j][b]);
#pragma unroll
            for (int r = 0; r < ROWS_TM; ++r) {
                float xv[V];
                Piece<T>::load(&x_s[r][i], xv);
#pragma unroll
                for (int j = 0; j < ROWS_J; ++j)
#pragma unroll
                    for (int b = 0; b < NB; ++b)
#pragma unroll
                        for (int e = 0; e < V; ++e) acc[j][b][r] += wv[j][b][e] * xv[e];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < ROWS_J; ++j) {
        const int col = col_base + warp + ROWS_WARPS * j;
#pragma unroll
        for (int r = 0; r < ROWS_TM; ++r) {
            float v = warp_sum(acc[j][0][r]);
            if (GATED) {
                const float g = to_float(from_float<T>(v)), u = to_float(from_float<T>(warp_sum(acc[j][NB - 1][r])));   // the projections' own rounding
                v = g / (1.0f + expf(-g)) * u;
            } else if (act >= 0) {
                v = mrs_activate(v, act);
            }
            const int pair = row_of[r];
            if (lane == 0 && col < n && pair >= 0) out[(size_t)(GATED || act >= 0 ? row0 + r : pair) * n + col] = from_float<T>(v);
        }
    }
}

// One block a listed row: sixteen bytes a thread and step.
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ sorted_rows, bf16* __restrict__ out, int k, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = sorted_rows[blockIdx.x];
    const uint4* src = pair >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)(pair / top) * k) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * k);
    for (int i = threadIdx.x; i < k / 8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

// The same with every row multiplied by its pair's weight (float32 product, rounded once), any size and both dtypes.
template <typename T>
__global__ void moe_gather_scaled_rows_kernel(const T* __restrict__ x, const int* __restrict__ sorted_rows, const float* __restrict__ weights,
                                              T* __restrict__ out, int k, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int pair = sorted_rows[blockIdx.x];
    const T* src = x + (size_t)(pair < 0 ? 0 : pair / top) * k;
    const float w = pair >= 0 ? weights[pair] : 0.0f;
    T* dst = out + (size_t)blockIdx.x * k;
    for (int i = threadIdx.x; i < k; i += blockDim.x) dst[i] = from_float<T>(pair >= 0 ? to_float(src[i]) * w : 0.0f);
}

// One block a token.  O: the sums leave as T, or as float32 (for a float32 norm or residual sum that reads them).
template <typename T, typename O>
__global__ void moe_combine_kernel(const T* __restrict__ y, const T* __restrict__ h, const T* __restrict__ shared_out,
                                   const int* __restrict__ chosen, const float* __restrict__ weights, const float* __restrict__ shared_gate,
                                   O* __restrict__ out, int width, int top, int routed) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float gate = shared_out ? (shared_gate ? shared_gate[t] : 1.0f) : 0.0f;        // no gates: the shared expert counts fully
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = 0.0f;
        for (int c = 0; c < top; ++c) {
            const int pair = t * top + c;
            const float part = chosen[pair] < routed ? to_float(y[(size_t)pair * width + i]) : to_float(h[(size_t)t * width + i]);
            v += (weights ? weights[pair] : 1.0f) * part;                                  // no weights: they were applied before
        }
        if (shared_out) v += gate * to_float(shared_out[(size_t)t * width + i]);
        out[(size_t)t * width + i] = from_float<O>(v);
    }
}

// The same, sixteen bytes a thread and step (width a multiple of 16 bytes, every row on a 16-byte boundary).
template <typename T> struct Store16;
template <> struct Store16<float> {
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Store16<bf16> {
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&two);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// The weighted gather with sixteen bytes a thread and step: k a multiple of 16 bytes, x and out on 16-byte boundaries.
template <typename T>
__global__ void moe_gather_scaled_rows_vec_kernel(const T* __restrict__ x, const int* __restrict__ sorted_rows, const float* __restrict__ weights,
                                                  T* __restrict__ out, int k, int top) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int V = Piece<T>::N;
    const int pair = sorted_rows[blockIdx.x];
    const T* src = x + (size_t)(pair < 0 ? 0 : pair / top) * k;
    const float w = pair >= 0 ? weights[pair] : 0.0f;
    T* dst = out + (size_t)blockIdx.x * k;
    for (int i = threadIdx.x * V; i < k; i += blockDim.x * V) {
        float v[V] = {};
        if (pair >= 0) {
            Piece<T>::load(src + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) v[e] *= w;
        }
        Store16<T>::store(dst + i, v);
    }
}

template <typename T, typename O>
__global__ void moe_combine_vec_kernel(const T* __restrict__ y, const T* __restrict__ h, const T* __restrict__ shared_out,
                                       const int* __restrict__ chosen, const float* __restrict__ weights, const float* __restrict__ shared_gate,
                                       O* __restrict__ out, int width, int top, int routed) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int V = Piece<T>::N;
    const int t = blockIdx.x;
    const float gate = shared_out ? (shared_gate ? shared_gate[t] : 1.0f) : 0.0f;        // no gates: the shared expert counts fully
    for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
        float v[V] = {};
        float own[V];
        bool have_own = false;
        for (int c = 0; c < top; ++c) {
            const int pair = t * top + c;
            const float weight = weights ? weights[pair] : 1.0f;
            float part[V];
            if (chosen[pair] < routed) {
                Piece<T>::load(y + (size_t)pair * width + i, part);
            } else {
                if (!have_own) Piece<T>::load(h + (size_t)t * width + i, own), have_own = true;
#pragma unroll
                for (int e = 0; e < V; ++e) part[e] = own[e];
            }
#pragma unroll
            for (int e = 0; e < V; ++e) v[e] += weight * part[e];
        }
        if (shared_out) {
            float part[V];
            Piece<T>::load(shared_out + (size_t)t * width + i, part);
#pragma unroll
            for (int e = 0; e < V; ++e) v[e] += gate * part[e];
        }
        if (sizeof(O) == sizeof(T)) {
            Store16<T>::store(reinterpret_cast<T*>(out) + (size_t)t * width + i, v);
        } else {                                   // float32 sums of bfloat16 parts: eight floats, two stores
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)t * width + i);
#pragma unroll
            for (int e = 0; e < V / 4; ++e) dst[e] = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
        }
    }
}

}  // namespace

MRS_EXPORT int mrs_moe_simt_tile() { return SIMT_TM; }

MRS_EXPORT int mrs_moe_route(const float* logits, int stride, const float* correction, int* chosen, float* weights, float* shared_gate,
                             int tokens, int all, int top, float scale, int sigmoid_scores, int has_shared, int normalize, void* stream) {
    if (tokens <= 0) return 0;
    if (all <= 0 || top <= 0 || top > all || stride < all + (has_shared ? 1 : 0) || (has_shared && !shared_gate)) return MRS_BAD_ARGUMENT;
    int warps = 4;
    while (warps > 1 && (size_t)warps * 2 * all * sizeof(float) > 40 * 1024) warps >>= 1;
    const size_t smem = (size_t)warps * 2 * all * sizeof(float);
    if (smem > 48 * 1024) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(moe_route_kernel, (tokens + warps - 1) / warps, 32 * warps, smem, stream, logits, stride, correction, chosen, weights,
               shared_gate, tokens, all, top, scale, sigmoid_scores, has_shared, normalize);
    MRS_RETURN_LAUNCH_STATUS();
}

// Rows of the lists for `pairs` pairs over `routed` experts in tiles of `tile` rows.
MRS_EXPORT long long mrs_moe_capacity(int pairs, int routed, int tile) {
    const long long most = (long long)pairs + (long long)routed * (tile - 1);
    return (most + tile - 1) / tile * tile;
}

MRS_EXPORT int mrs_moe_align(const int* chosen, int pairs, int routed, int tile, int* sorted_rows, int* tile_expert, int capacity,
                             void* stream) {
    if (pairs <= 0) return 0;
    if (routed <= 0 || tile <= 0 || capacity % tile || capacity < mrs_moe_capacity(pairs, routed, tile) || routed > 4096) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(moe_align_kernel, 1, 1024, (size_t)3 * routed * sizeof(int), stream, chosen, pairs, routed, tile, sorted_rows, tile_expert,
               capacity);
    MRS_RETURN_LAUNCH_STATUS();
}

// gated != 0: x [tokens, k], weight [experts, 2 n, k], out [capacity, n]; else x [capacity, k], weight [experts, n, k],
// out [pairs, n], or with act >= 0 (an activation's number) out [capacity, n] = activation of the sums, at the rows' places.
// Lists in tiles of mrs_moe_simt_tile() rows.  `block` > 0 (gated): gate and up rows alternate in blocks.
MRS_EXPORT int mrs_moe_product_simt(int is_bf16, int gated, const void* x, const int* sorted_rows, const int* tile_expert,
                                    const void* weight, void* out, int capacity, int n, int k, int top, int block, int act, void* stream) {
    if (capacity <= 0) return 0;
    if (capacity % SIMT_TM || n <= 0 || k <= 0 || top <= 0 || block < 0 || (block && n % block) || act > 4 || (gated && act >= 0))
        return MRS_BAD_ARGUMENT;
    const dim3 grid(capacity / SIMT_TM, (n + SIMT_TN - 1) / SIMT_TN);
#define MRS_MOE_SIMT(T, GATED)                                                                                                   \
    MRS_LAUNCH((moe_product_simt_kernel<T, GATED>), grid, 256, 0, stream, (const T*)x, sorted_rows, tile_expert, (const T*)weight, \
               (T*)out, n, k, top, block, act)
    if (is_bf16) {
        if (gated) MRS_MOE_SIMT(bf16, true); else MRS_MOE_SIMT(bf16, false);
    } else {
        if (gated) MRS_MOE_SIMT(float, true); else MRS_MOE_SIMT(float, false);
    }
#undef MRS_MOE_SIMT
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_moe_rows_tile() { return ROWS_TM; }

// As mrs_moe_product_simt for lists in tiles of mrs_moe_rows_tile() rows: few rows an expert.  k * sizeof(T) a multiple of 16,
// x, weight on 16-byte boundaries.
MRS_EXPORT int mrs_moe_product_rows(int is_bf16, int gated, const void* x, const int* sorted_rows, const int* tile_expert,
                                    const void* weight, void* out, int capacity, int n, int k, int top, int block, int act, void* stream) {
    if (capacity <= 0) return 0;
    if (capacity % ROWS_TM || n <= 0 || k <= 0 || k % (is_bf16 ? 8 : 4) || top <= 0 || block < 0 || (block && (!gated || n % block)) ||
        act > 4 || (gated && act >= 0) ||
        (((uintptr_t)x | (uintptr_t)weight) & 15))
        return MRS_BAD_ARGUMENT;
    const dim3 grid(capacity / ROWS_TM, (n + ROWS_WARPS * ROWS_J - 1) / (ROWS_WARPS * ROWS_J));
#define MRS_MOE_ROWS(T, GATED)                                                                                                             \
    MRS_LAUNCH((moe_product_rows_kernel<T, GATED>), grid, 32 * ROWS_WARPS, 0, stream, (const T*)x, sorted_rows, tile_expert, (const T*)weight, \
               (T*)out, n, k, top, block, act)
    if (is_bf16) {
        if (gated) MRS_MOE_ROWS(bf16, true); else MRS_MOE_ROWS(bf16, false);
    } else {
        if (gated) MRS_MOE_ROWS(float, true); else MRS_MOE_ROWS(float, false);
    }
#undef MRS_MOE_ROWS
    MRS_RETURN_LAUNCH_STATUS();
}

// out [capacity, k] = the input rows x[pair / top] of the listed pairs, zeros for -1; bfloat16, k a multiple of 8.
MRS_EXPORT int mrs_moe_gather_rows(const void* x, const int* sorted_rows, void* out, int capacity, int k, int top, void* stream) {
    if (capacity <= 0) return 0;
    if (k <= 0 || k % 8 || top <= 0 || (((uintptr_t)x | (uintptr_t)out) & 15)) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(moe_gather_rows_kernel, capacity, 128, 0, stream, (const bf16*)x, sorted_rows, (bf16*)out, k, top);
    MRS_RETURN_LAUNCH_STATUS();
}

// out [capacity, k] = x[pair / top] * weights[pair] for the listed pairs, zeros for -1; any k, both dtypes.
MRS_EXPORT int mrs_moe_gather_scaled_rows(int is_bf16, const void* x, const int* sorted_rows, const float* weights, void* out, int capacity,
                                          int k, int top, void* stream) {
    if (capacity <= 0) return 0;
    if (k <= 0 || top <= 0 || !weights) return MRS_BAD_ARGUMENT;
    if (k % (is_bf16 ? 8 : 4) == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        if (is_bf16)
            MRS_LAUNCH(moe_gather_scaled_rows_vec_kernel<bf16>, capacity, 128, 0, stream, (const bf16*)x, sorted_rows, weights, (bf16*)out, k, top);
        else
            MRS_LAUNCH(moe_gather_scaled_rows_vec_kernel<float>, capacity, 128, 0, stream, (const float*)x, sorted_rows, weights, (float*)out, k, top);
        MRS_RETURN_LAUNCH_STATUS();
    }
    if (is_bf16)
        MRS_LAUNCH(moe_gather_scaled_rows_kernel<bf16>, capacity, 128, 0, stream, (const bf16*)x, sorted_rows, weights, (bf16*)out, k, top);
    else
        MRS_LAUNCH(moe_gather_scaled_rows_kernel<float>, capacity, 128, 0, stream, (const float*)x, sorted_rows, weights, (float*)out, k, top);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_moe_combine(int is_bf16, const void* y, const void* h, const void* shared_out, const int* chosen, const float* weights,
                               const float* shared_gate, void* out, int tokens, int width, int top, int routed, int out_float32, void* stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || top <= 0) return MRS_BAD_ARGUMENT;
    const int threads = width >= 1024 ? 256 : 128;
    const bool aligned = (((uintptr_t)y | (uintptr_t)h | (uintptr_t)shared_out | (uintptr_t)out) & 15) == 0;
    const bool vec = aligned && width % (is_bf16 ? 8 : 4) == 0;
#define MRS_MOE_COMBINE(T, O)                                                                                                          \
    do {                                                                                                                               \
        if (vec)                                                                                                                       \
            MRS_LAUNCH((moe_combine_vec_kernel<T, O>), tokens, 128, 0, stream, (const T*)y, (const T*)h, (const T*)shared_out, chosen,   \
                       weights, shared_gate, (O*)out, width, top, routed);                                                             \
        else                                                                                                                           \
            MRS_LAUNCH((moe_combine_kernel<T, O>), tokens, threads, 0, stream, (const T*)y, (const T*)h, (const T*)shared_out, chosen,   \
                       weights, shared_gate, (O*)out, width, top, routed);                                                             \
    } while (0)
    if (!is_bf16) MRS_MOE_COMBINE(float, float);
    else if (out_float32) MRS_MOE_COMBINE(bf16, float);
    else MRS_MOE_COMBINE(bf16, bf16);
#undef MRS_MOE_COMBINE
    MRS_RETURN_LAUNCH_STATUS();
}
