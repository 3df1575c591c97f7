// Row-wise kernels of layers that norm a branch before it joins the stream, clamp a gated
// feed-forward, add biases to q/k/v and blend values between layers, and norm a gated
// recurrence output in parts.  All statistics, sums and gates are float32; T is the engine's
// dtype (float or bfloat16) and is only what a kernel hands to the next product or the cache.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// stream += mult * rmsnorm(branch) * w_post;  out = rmsnorm(stream) * w_next   (w_next may be null: sum only)
// branch float32 [rows, width] (a product's float32 sums), stream float32, out T.
// One block a row; the row is read three times from L1/L2.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void postnorm_add_norm_kernel(float* __restrict__ stream, const float* __restrict__ branch,
                                         const float* __restrict__ w_post, const float* __restrict__ w_next, float eps_post,
                                         float eps_next, T* __restrict__ out, int width, float mult) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    float* res = stream + r * width;
    const float* a = branch + r * width;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) sum += a[i] * a[i];
    const float scale_a = mult / sqrtf(block_sum(sum, scratch) / (float)width + eps_post);
    sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = res[i] + a[i] * scale_a * w_post[i];
        res[i] = v;
        sum += v * v;
    }
    if (w_next == nullptr) return;
    const float scale_v = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps_next);
    T* o = out + r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_float<T>(res[i] * scale_v * w_next[i]);
}

// The same with the row kept in registers between the passes and four elements a load: width a multiple of 4, at most
// 16 * blockDim.x, rows on 16-byte boundaries.  Every element is read once.
#define NORM_KEEP 4
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

template <typename T>
__global__ void postnorm_add_norm_kept_kernel(float* __restrict__ stream, const float* __restrict__ branch,
                                              const float* __restrict__ w_post, const float* __restrict__ w_next, float eps_post,
                                              float eps_next, T* __restrict__ out, int width, float mult) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    float* res = stream + r * width;
    const float* a = branch + r * width;
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 av[NORM_KEEP], rv[NORM_KEEP], wv[NORM_KEEP];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        av[j] = i < width ? ld4(a + i) : zero;
        sum += av[j].x * av[j].x + av[j].y * av[j].y + av[j].z * av[j].z + av[j].w * av[j].w;
    }
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {                  // asked for before the block waits for its sum
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        rv[j] = i < width ? ld4(res + i) : zero;
        wv[j] = i < width ? ld4(w_post + i) : zero;
    }
    const float scale_a = mult / sqrtf(block_sum(sum, scratch) / (float)width + eps_post);
    sum = 0.0f;
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < width) {
            rv[j].x += av[j].x * scale_a * wv[j].x, rv[j].y += av[j].y * scale_a * wv[j].y;
            rv[j].z += av[j].z * scale_a * wv[j].z, rv[j].w += av[j].w * scale_a * wv[j].w;
            st4<float>(res + i, rv[j]);
            sum += rv[j].x * rv[j].x + rv[j].y * rv[j].y + rv[j].z * rv[j].z + rv[j].w * rv[j].w;
        }
    }
    if (w_next == nullptr) return;
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        wv[j] = i < width ? ld4(w_next + i) : zero;
    }
    const float scale_v = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps_next);
    T* o = out + r * width;
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < width)
            st4<T>(o + i, make_float4(rv[j].x * scale_v * wv[j].x, rv[j].y * scale_v * wv[j].y, rv[j].z * scale_v * wv[j].z,
                                      rv[j].w * scale_v * wv[j].w));
    }
}

MRS_EXPORT int mrs_postnorm_add_norm(int is_bf16, float* stream, const float* branch, const float* w_post, const float* w_next,
                                     float eps_post, float eps_next, void* out, int rows, int width, float mult, void* s) {
    if (rows <= 0) return 0;
    if (width <= 0) return MRS_BAD_ARGUMENT;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const bool aligned = (((uintptr_t)stream | (uintptr_t)branch | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && aligned && width <= 4 * NORM_KEEP * 512) {
        int kept_threads = ((width / 4 + NORM_KEEP - 1) / NORM_KEEP + 31) / 32 * 32;      // the row fits the block's registers
        if (kept_threads < 64) kept_threads = 64;
        if (is_bf16)
            MRS_LAUNCH(postnorm_add_norm_kept_kernel<bf16>, rows, kept_threads, 0, s, stream, branch, w_post, w_next, eps_post, eps_next, (bf16*)out, width, mult);
        else
            MRS_LAUNCH(postnorm_add_norm_kept_kernel<float>, rows, kept_threads, 0, s, stream, branch, w_post, w_next, eps_post, eps_next, (float*)out, width, mult);
        MRS_RETURN_LAUNCH_STATUS();
    }
    if (is_bf16)
        MRS_LAUNCH(postnorm_add_norm_kernel<bf16>, rows, threads, 0, s, stream, branch, w_post, w_next, eps_post, eps_next, (bf16*)out, width, mult);
    else
        MRS_LAUNCH(postnorm_add_norm_kernel<float>, rows, threads, 0, s, stream, branch, w_post, w_next, eps_post, eps_next, (float*)out, width, mult);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// Clamped gated unit: g = min(gate, limit), u = clamp(up, -limit, limit); out = g * sigmoid(alpha g) * (u + 1).
// gate_up [tokens, 2 * inter]: all gate columns, then all up columns.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int tokens, int inter, float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    // a thread keeps its two columns and walks down the tokens: no division, neighbouring threads read neighbouring pairs
    const int c = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (c >= inter) return;
    const bool pair = c + 1 < inter;
    for (int t = blockIdx.y; t < tokens; t += gridDim.y) {
        const T* row = gate_up + (size_t)t * 2 * inter;
        T* o = out + (size_t)t * inter;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (j == 1 && !pair) break;
            const float g = fminf(to_float(row[c + j]), limit);
            const float u = fminf(fmaxf(to_float(row[inter + c + j]), -limit), limit);
            o[c + j] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
        }
    }
}

MRS_EXPORT int mrs_glu_clamped(int is_bf16, const void* gate_up, void* out, int tokens, int inter, float limit, float alpha, void* s) {
    if (tokens <= 0 || inter <= 0) return 0;
    const int threads = 128;
    const unsigned across = (unsigned)((inter + 2 * threads - 1) / (2 * threads));
    long long down = ((long long)mrs_sm_count() * 32 + across - 1) / across;
    if (down > tokens) down = tokens;
    if (down > 65535) down = 65535;
    if (is_bf16)
        MRS_LAUNCH(glu_clamped_kernel<bf16>, dim3(across, (unsigned)down), threads, 0, s, (const bf16*)gate_up, (bf16*)out, tokens, inter, limit, alpha);
    else
        MRS_LAUNCH(glu_clamped_kernel<float>, dim3(across, (unsigned)down), threads, 0, s, (const float*)gate_up, (float*)out, tokens, inter, limit, alpha);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// After the fused q|k|v|gate projection (float32 sums [tokens, nq*d + nkv*d + nkv*e + nq]):
// adds the biases of q, k and v; q -> q_out (T); k -> key pages; v, blended with the values that an
// earlier layer left for the same token (v <- (1 - lambda) v + lambda v_first), -> value pages;
// sigmoid of the gate columns -> gate_out float32 [tokens, nq].
// mix_mode 0: no blending; 1: this layer's own values (with bias) are written to v_first; 2: blend from v_first.
// Key pages [pages, nkv, page, d], value pages [pages, nkv, page, e]; slot < 0 writes nothing.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void qkv_bias_store_kernel(const float* __restrict__ proj, const float* __restrict__ bias, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
                                      float* __restrict__ v_first, float* __restrict__ gate_out, int nq, int nkv, int d, int e,
                                      int page_size, int mix_mode, float lambda, int has_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int qw = nq * d, kw = nkv * d, vw = nkv * e;
    const int total = qw + kw + vw + (has_gate ? nq : 0);
    const float* row = proj + t * total;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, in_page = slot >= 0 ? slot % page_size : 0;
    for (int c = threadIdx.x; c < total; c += blockDim.x) {
        if (c < qw) {
            q_out[t * qw + c] = from_float<T>(row[c] + (bias ? bias[c] : 0.0f));
        } else if (c < qw + kw) {
            const int j = c - qw, head = j / d, x = j % d;
            if (slot >= 0 && k_cache)
                k_cache[(((size_t)page * nkv + head) * page_size + in_page) * d + x] = from_float<T>(row[c] + (bias ? bias[c] : 0.0f));
        } else if (c < qw + kw + vw) {
            const int j = c - qw - kw, head = j / e, x = j % e;
            float v = row[c] + (bias ? bias[c] : 0.0f);
            if (mix_mode == 1) v_first[t * vw + j] = v;
            else if (mix_mode == 2) v = (1.0f - lambda) * v + lambda * v_first[t * vw + j];
            if (slot >= 0 && v_cache)
                v_cache[(((size_t)page * nkv + head) * page_size + in_page) * e + x] = from_float<T>(v);
        } else {
            const int h = c - qw - kw - vw;
            gate_out[t * nq + h] = 1.0f / (1.0f + expf(-row[c]));
        }
    }
}

// The same with an RMS norm over every query and key head before it leaves (weights q_norm, k_norm [d] float32, shared by
// the heads; x / sqrt(mean(x^2) + eps) * w after the bias): one warp a head, so that a head's sum of squares is a few
// shuffles.  No blending of values.
template <typename T>
__global__ void qkv_headnorm_store_kernel(const float* __restrict__ proj, const float* __restrict__ bias, const float* __restrict__ q_norm,
                                          const float* __restrict__ k_norm, float eps, T* __restrict__ q_out, T* __restrict__ k_cache,
                                          T* __restrict__ v_cache, const int* __restrict__ slots, float* __restrict__ gate_out, int nq,
                                          int nkv, int d, int e, int page_size, int has_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int qw = nq * d, kw = nkv * d, vw = nkv * e;
    const int total = qw + kw + vw + (has_gate ? nq : 0);
    const float* row = proj + t * total;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, in_page = slot >= 0 ? slot % page_size : 0;
    for (int unit = warp; unit < nq + 2 * nkv; unit += warps) {
        if (unit < nq + nkv) {                               // a query or key head
            const bool is_q = unit < nq;
            const int head = is_q ? unit : unit - nq, at = is_q ? head * d : qw + head * d;
            const float* w = is_q ? q_norm : k_norm;
            if (!is_q && (slot < 0 || !k_cache)) continue;
            float sum = 0.0f;
            for (int x = lane; x < d; x += 32) {
                const float v = row[at + x] + (bias ? bias[at + x] : 0.0f);
                sum += v * v;
            }
            const float scale = w ? 1.0f / sqrtf(warp_sum(sum) / (float)d + eps) : 1.0f;
            T* dst = is_q ? q_out + t * qw + (size_t)head * d : k_cache + (((size_t)page * nkv + head) * page_size + in_page) * d;
            for (int x = lane; x < d; x += 32) {
                const float v = row[at + x] + (bias ? bias[at + x] : 0.0f);
                dst[x] = from_float<T>(w ? v * scale * w[x] : v);
            }
        } else if (slot >= 0 && v_cache) {                   // a value head
            const int head = unit - nq - nkv, at = qw + kw + head * e;
            T* dst = v_cache + (((size_t)page * nkv + head) * page_size + in_page) * e;
            for (int x = lane; x < e; x += 32) dst[x] = from_float<T>(row[at + x] + (bias ? bias[at + x] : 0.0f));
        }
    }
    if (has_gate)
        for (int h = threadIdx.x; h < nq; h += blockDim.x) gate_out[t * nq + h] = 1.0f / (1.0f + expf(-row[qw + kw + vw + h]));
}

MRS_EXPORT int mrs_qkv_bias_store(int is_bf16, const float* proj, const float* bias, void* q_out, void* k_cache, void* v_cache,
                                  const int* slots, float* v_first, float* gate_out, int tokens, int nq, int nkv, int d, int e,
                                  int page_size, int mix_mode, float lambda, int has_gate, const float* q_norm, const float* k_norm,
                                  float norm_eps, void* s) {
    if (tokens <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || d <= 0 || e <= 0 || page_size <= 0 || (mix_mode && !v_first) || (has_gate && !gate_out) ||
        ((q_norm || k_norm) && mix_mode))
        return MRS_BAD_ARGUMENT;
    if (q_norm || k_norm) {
        const int units = nq + 2 * nkv;
        const int threads = units >= 8 ? 256 : (units >= 4 ? 128 : 64);
        if (is_bf16)
            MRS_LAUNCH(qkv_headnorm_store_kernel<bf16>, tokens, threads, 0, s, proj, bias, q_norm, k_norm, norm_eps, (bf16*)q_out,
                       (bf16*)k_cache, (bf16*)v_cache, slots, gate_out, nq, nkv, d, e, page_size, has_gate);
        else
            MRS_LAUNCH(qkv_headnorm_store_kernel<float>, tokens, threads, 0, s, proj, bias, q_norm, k_norm, norm_eps, (float*)q_out,
                       (float*)k_cache, (float*)v_cache, slots, gate_out, nq, nkv, d, e, page_size, has_gate);
        MRS_RETURN_LAUNCH_STATUS();
    }
    if (is_bf16)
        MRS_LAUNCH(qkv_bias_store_kernel<bf16>, tokens, 256, 0, s, proj, bias, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, slots,
                   v_first, gate_out, nq, nkv, d, e, page_size, mix_mode, lambda, has_gate);
    else
        MRS_LAUNCH(qkv_bias_store_kernel<float>, tokens, 256, 0, s, proj, bias, (float*)q_out, (float*)k_cache, (float*)v_cache, slots,
                   v_first, gate_out, nq, nkv, d, e, page_size, mix_mode, lambda, has_gate);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// out = rmsnorm_in_parts(y * silu(z)) * weight: the row of `inner` elements is cut into `parts` equal parts,
// each divided by its own root mean square.  y float32 [tokens, inner]; z float32, a column range of a wider
// row (z_stride elements a row); out T [tokens, inner].  One block a (token, part).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_part_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, int z_stride,
                                       const float* __restrict__ weight, float eps, T* __restrict__ out, int inner, int parts) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const int part = blockIdx.y, width = inner / parts, first = part * width;
    const float* yr = y + t * inner + first;
    const float* zr = z + t * z_stride + first;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float g = yr[i] * (zr[i] / (1.0f + expf(-zr[i])));
        sum += g * g;
    }
    const float scale = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps);
    T* o = out + t * inner + first;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float g = yr[i] * (zr[i] / (1.0f + expf(-zr[i])));
        o[i] = from_float<T>(g * scale * weight[first + i]);
    }
}

MRS_EXPORT int mrs_gated_part_norm(int is_bf16, const float* y, const float* z, int z_stride, const float* weight, float eps,
                                   void* out, int tokens, int inner, int parts, void* s) {
    if (tokens <= 0) return 0;
    if (parts <= 0 || inner <= 0 || inner % parts) return MRS_BAD_ARGUMENT;
    const int width = inner / parts;
    const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
    if (is_bf16)
        MRS_LAUNCH(gated_part_norm_kernel<bf16>, dim3(tokens, parts), threads, 0, s, y, z, z_stride, weight, eps, (bf16*)out, inner, parts);
    else
        MRS_LAUNCH(gated_part_norm_kernel<float>, dim3(tokens, parts), threads, 0, s, y, z, z_stride, weight, eps, (float*)out, inner, parts);
    MRS_RETURN_LAUNCH_STATUS();
}
