// Row-wise kernels of layers whose branches run side by side on one normed input, of plain (ungated) feed-forwards and
// of capped logits.  Sums, statistics and the activation's arithmetic are float32; T is the engine's dtype.
//
//   add_branches_norm   stream += a (+ b);  out = stream / sqrt(mean(stream^2) + eps) * w_next   (w_next may be null: sum only)
//   activation          out = act(in):  0 = gelu with the error function, 0.5 z (1 + erf(z / sqrt 2));
//                                       1 = gelu with tanh, 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)));   2 = silu
//   scale_softcap       x <- cap * tanh(x * scale / cap)
#include "common.cuh"

namespace {

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// Any width: one block a row, the sum is written and read again for the norm.
template <typename T>
__global__ void add_branches_norm_kernel(float* __restrict__ stream, const float* __restrict__ a, const float* __restrict__ b,
                                         const float* __restrict__ w_next, float eps, T* __restrict__ out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    float* res = stream + r * width;
    const float* ar = a + r * width;
    const float* br = b ? b + r * width : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = res[i] + (br ? ar[i] + br[i] : ar[i]);
        res[i] = v;
        sum += v * v;
    }
    if (w_next == nullptr) return;
    const float scale = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps);
    T* o = out + r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_float<T>(res[i] * scale * w_next[i]);
}

// Width a multiple of 4, at most 16 * blockDim.x, rows on 16-byte boundaries: the row stays in registers between the
// passes and every element is read once, four a load.
#define BRANCH_KEEP 4
template <typename T>
__global__ void add_branches_norm_kept_kernel(float* __restrict__ stream, const float* __restrict__ a, const float* __restrict__ b,
                                              const float* __restrict__ w_next, float eps, T* __restrict__ out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    float* res = stream + r * width;
    const float* ar = a + r * width;
    const float* br = b ? b + r * width : nullptr;
    float4 v[BRANCH_KEEP], w[BRANCH_KEEP];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < BRANCH_KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < width) {
            v[j] = ld4(res + i);
            float4 x = ld4(ar + i);
            if (br) {
                const float4 y = ld4(br + i);
                x.x += y.x, x.y += y.y, x.z += y.z, x.w += y.w;
            }
            v[j].x += x.x, v[j].y += x.y, v[j].z += x.z, v[j].w += x.w;
            st4<float>(res + i, v[j]);
            sum += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    if (w_next == nullptr) return;
#pragma unroll
    for (int j = 0; j < BRANCH_KEEP; ++j) {                  // asked for before the block waits for its sum
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        w[j] = i < width ? ld4(w_next + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    const float scale = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps);
    T* o = out + r * width;
#pragma unroll
    for (int j = 0; j < BRANCH_KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < width)
            st4<T>(o + i, make_float4(v[j].x * scale * w[j].x, v[j].y * scale * w[j].y, v[j].z * scale * w[j].z, v[j].w * scale * w[j].w));
    }
}

__device__ __forceinline__ float activate(float z, int kind) {
    if (kind == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));
    if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    if (kind == 3) return fmaxf(z, 0.0f);
    if (kind == 4) return fmaxf(z, 0.0f) * fmaxf(z, 0.0f);
    return z / (1.0f + expf(-z));
}

// A gated unit's inner rows: out = act(gate) * up over `gate_up` [tokens, 2 * inter]: all gate columns and then all up
// columns (block 0), or blocks of `block` gate columns each followed by the matching up columns (inter a multiple of
// block).  A thread keeps its two columns and walks down the tokens.
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int tokens, int inter, int kind, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (c >= inter) return;
    const bool pair = c + 1 < inter;
    const int g0 = block ? c / block * 2 * block + c % block : c, u0 = g0 + (block ? block : inter);
    const int g1 = block ? (c + 1) / block * 2 * block + (c + 1) % block : c + 1, u1 = g1 + (block ? block : inter);
    for (int t = blockIdx.y; t < tokens; t += gridDim.y) {
        const T* row = gate_up + (size_t)t * 2 * inter;
        T* o = out + (size_t)t * inter;
        o[c] = from_float<T>(activate(to_float(row[g0]), kind) * to_float(row[u0]));
        if (pair) o[c + 1] = from_float<T>(activate(to_float(row[g1]), kind) * to_float(row[u1]));
    }
}

template <typename T>
__global__ void activation_kernel(const T* in, T* out, long long n, int kind) {      // out may be in
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = from_float<T>(activate(to_float(in[i]), kind));
}

// Eight bfloat16 (16 bytes) a thread and trip; n a multiple of 8, both pointers on 16-byte boundaries.
__global__ void activation_bf16x8_kernel(const uint4* in, uint4* out, long long n8, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        uint4 raw = in[i];
        uint32_t* words = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 z = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&words[j]));
            __nv_bfloat162 y = __floats2bfloat162_rn(activate(z.x, kind), activate(z.y, kind));
            words[j] = *reinterpret_cast<uint32_t*>(&y);
        }
        out[i] = raw;
    }
}

__global__ void scale_softcap_kernel(float* __restrict__ x, long long n, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const float inside = scale / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inside);
}

}  // namespace

MRS_EXPORT int mrs_add_branches_norm(int is_bf16, float* stream, const float* a, const float* b, const float* w_next, float eps,
                                     void* out, int rows, int width, void* s) {
    if (rows <= 0) return 0;
    if (width <= 0 || !a || (w_next && !out)) return MRS_BAD_ARGUMENT;
    const bool aligned = (((uintptr_t)stream | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && aligned && width <= 4 * BRANCH_KEEP * 512) {
        int threads = ((width / 4 + BRANCH_KEEP - 1) / BRANCH_KEEP + 31) / 32 * 32;
        if (threads < 64) threads = 64;
        if (is_bf16)
            MRS_LAUNCH(add_branches_norm_kept_kernel<bf16>, rows, threads, 0, s, stream, a, b, w_next, eps, (bf16*)out, width);
        else
            MRS_LAUNCH(add_branches_norm_kept_kernel<float>, rows, threads, 0, s, stream, a, b, w_next, eps, (float*)out, width);
        MRS_RETURN_LAUNCH_STATUS();
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (is_bf16)
        MRS_LAUNCH(add_branches_norm_kernel<bf16>, rows, threads, 0, s, stream, a, b, w_next, eps, (bf16*)out, width);
    else
        MRS_LAUNCH(add_branches_norm_kernel<float>, rows, threads, 0, s, stream, a, b, w_next, eps, (float*)out, width);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_activation(int is_bf16, const void* in, void* out, long long n, int kind, void* s) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 4) return MRS_BAD_ARGUMENT;
    const int threads = 256;
    const long long cap = 16LL * mrs_sm_count();
    if (is_bf16 && n % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        long long blocks = (n / 8 + threads - 1) / threads;
        if (blocks > cap) blocks = cap;
        MRS_LAUNCH(activation_bf16x8_kernel, (unsigned)blocks, threads, 0, s, (const uint4*)in, (uint4*)out, n / 8, kind);
        MRS_RETURN_LAUNCH_STATUS();
    }
    long long blocks = (n + threads - 1) / threads;
    if (blocks > cap) blocks = cap;
    if (is_bf16)
        MRS_LAUNCH(activation_kernel<bf16>, (unsigned)blocks, threads, 0, s, (const bf16*)in, (bf16*)out, n, kind);
    else
        MRS_LAUNCH(activation_kernel<float>, (unsigned)blocks, threads, 0, s, (const float*)in, (float*)out, n, kind);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_gated_activation(int is_bf16, const void* gate_up, void* out, int tokens, int inter, int kind, int block, void* s) {
    if (tokens <= 0 || inter <= 0) return 0;
    if (kind < 0 || kind > 4 || block < 0 || (block > 0 && inter % block)) return MRS_BAD_ARGUMENT;
    const int threads = 128;
    const unsigned across = (unsigned)((inter + 2 * threads - 1) / (2 * threads));
    long long down = ((long long)mrs_sm_count() * 32 + across - 1) / across;
    if (down > tokens) down = tokens;
    if (down > 65535) down = 65535;
    if (is_bf16)
        MRS_LAUNCH(gated_activation_kernel<bf16>, dim3(across, (unsigned)down), threads, 0, s, (const bf16*)gate_up, (bf16*)out, tokens, inter, kind, block);
    else
        MRS_LAUNCH(gated_activation_kernel<float>, dim3(across, (unsigned)down), threads, 0, s, (const float*)gate_up, (float*)out, tokens, inter, kind, block);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_scale_softcap(float* x, long long n, float scale, float cap, void* s) {
    if (n <= 0) return 0;
    if (!(cap > 0.0f)) return MRS_BAD_ARGUMENT;
    long long blocks = (n + 255) / 256;
    if (blocks > 8LL * mrs_sm_count()) blocks = 8LL * mrs_sm_count();
    MRS_LAUNCH(scale_softcap_kernel, (unsigned)blocks, 256, 0, s, x, n, scale, cap);
    MRS_RETURN_LAUNCH_STATUS();
}
