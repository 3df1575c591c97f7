// Kernels around a latent attention and a layer norm with bias (every size at run time, float32 or bfloat16
// activations, statistics, angles and gates in float32):
//
//   add_layernorm     v = residual (+ delta);  out = (v - mean) / sqrt(var + eps) * weight + bias, var the mean of the
//                     squared deviations (computed from the mean, not from the mean of squares)
//   latent_prepare    what follows the fused projection q | latent, rotated key | gate of a latent attention:
//                     the unrotated query parts head-major for the product that carries them into the latent space,
//                     the rotated query parts behind the latent columns of the query rows, the latent divided by its
//                     root mean square and the rotated key part into the cache row of the token, sigmoid of the gates
//
//   latent_norms      for a latent attention whose queries pass a latent of their own and that rotates nothing: after the
//                     fused projection query latent | key/value latent | ..., both divided by their root mean squares times
//                     their weights; the first goes on to the queries' up-projection, the second into the cache row
//   sigmoid_gate_mul  x <- x * sigmoid(gate) element by element, the gate a column range of wider float32 rows
//
// Rotation: of the first `rotary` elements of a rotated part element i pairs with i + rotary / 2; the pair (u, v) at
// position p becomes (u c - v s, v c + u s) with c = m cos(p f_i), s = m sin(p f_i); the rest passes unchanged.
#include "common.cuh"

namespace {

#define LN_CHUNKS 4

template <typename T> struct Row4;
template <> struct Row4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Row4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// Any width: the row is read three times (sum, squared deviations, output).
template <typename T>
__global__ void add_layernorm_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ weight,
                                     const float* __restrict__ bias, float eps, T* __restrict__ out, const int* __restrict__ rows,
                                     int width, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * width;
    const T* del = delta ? delta + src * width : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del) v += to_float(del[i]);
        if (write_back && del) res[i] = v;
        sum += v;
    }
    const bool again = del && !write_back;         // the sum is not in memory: add the branch again
    const float mean = block_sum(sum, scratch) / (float)width;
    float dev = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = res[i] + (again ? to_float(del[i]) : 0.0f) - mean;
        dev += v * v;
    }
    const float scale = rsqrtf(block_sum(dev, scratch) / (float)width + eps);
    T* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = res[i] + (again ? to_float(del[i]) : 0.0f) - mean;
        o[i] = from_float<T>(v * scale * weight[i] + bias[i]);
    }
}

// Width a multiple of 4, at most 4 * LN_CHUNKS * blockDim.x: the row stays in registers between the passes.
template <typename T>
__global__ void add_layernorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ weight,
                                         const float* __restrict__ bias, float eps, T* __restrict__ out, const int* __restrict__ rows,
                                         int width, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * width;
    const T* del = delta ? delta + src * width : nullptr;
    float4 v[LN_CHUNKS];
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < LN_CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        v[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < width) {
            v[c] = Row4<float>::load(res + i);
            if (del) {
                const float4 d = Row4<T>::load(del + i);
                v[c].x += d.x, v[c].y += d.y, v[c].z += d.z, v[c].w += d.w;
                if (write_back) Row4<float>::store(res + i, v[c]);
            }
            sum += (v[c].x + v[c].y) + (v[c].z + v[c].w);
        }
    }
    const float mean = block_sum(sum, scratch) / (float)width;
    float dev = 0.0f;
#pragma unroll
    for (int c = 0; c < LN_CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < width) {
            v[c].x -= mean, v[c].y -= mean, v[c].z -= mean, v[c].w -= mean;
            dev += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
        }
    }
    const float scale = rsqrtf(block_sum(dev, scratch) / (float)width + eps);
    T* o = out + (size_t)r * width;
#pragma unroll
    for (int c = 0; c < LN_CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < width) {
            const float4 w = Row4<float>::load(weight + i), b = Row4<float>::load(bias + i);
            Row4<T>::store(o + i, make_float4(v[c].x * scale * w.x + b.x, v[c].y * scale * w.y + b.y, v[c].z * scale * w.z + b.z,
                                              v[c].w * scale * w.w + b.w));
        }
    }
}

__global__ void scale_kernel(float* __restrict__ x, long long n, float factor) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= factor;
}

struct LatentSizes {
    int heads, plain, rotated, latent, rotary;      // per head: unrotated and rotated query/key elements; latent size; rotated pairs * 2
    int has_latent, has_gate;
};

// One block a token.  Columns of a projected row: heads * (plain + rotated) of q, then (has_latent) latent + rotated,
// then (has_gate) one gate a head.  Dynamic shared memory: rotary floats (cosines, then sines).
template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ proj, int proj_width, const float* __restrict__ latent_weight, float eps,
                                      const float* __restrict__ inv_freq, float magnitude, const int* __restrict__ positions,
                                      const int* __restrict__ slots, T* __restrict__ q_plain, T* __restrict__ q_rows, T* __restrict__ cache,
                                      float* __restrict__ gate, int tokens, LatentSizes z) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float turn[];
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * proj_width;
    const int half = z.rotary / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        turn[i] = c * magnitude;
        turn[half + i] = s * magnitude;
    }
    __syncthreads();
    const int per_head = z.plain + z.rotated, key_width = z.latent + z.rotated;
    auto rotated_at = [&](const float* part, int i) {        // element i of a rotated part
        if (i >= z.rotary) return part[i];
        const int j = i < half ? i : i - half;
        const float u = part[j], v = part[j + half], c = turn[j], s = turn[half + j];
        return i < half ? u * c - v * s : v * c + u * s;
    };
    for (int idx = threadIdx.x; idx < z.heads * per_head; idx += blockDim.x) {
        const int h = idx / per_head, x = idx % per_head;
        if (x < z.plain)
            q_plain[((size_t)h * tokens + t) * z.plain + x] = from_float<T>(row[idx]);
        else
            q_rows[((size_t)t * z.heads + h) * key_width + z.latent + (x - z.plain)] =
                from_float<T>(rotated_at(row + h * per_head + z.plain, x - z.plain));
    }
    int at = z.heads * per_head;
    if (z.has_latent) {
        const float* low = row + at;
        float sum = 0.0f;
        for (int i = threadIdx.x; i < z.latent; i += blockDim.x) sum += low[i] * low[i];
        const float scale = rsqrtf(block_sum(sum, scratch) / (float)z.latent + eps);
        const int slot = slots ? slots[t] : -1;
        if (slot >= 0 && cache) {
            T* dst = cache + (size_t)slot * key_width;
            for (int i = threadIdx.x; i < key_width; i += blockDim.x)
                dst[i] = from_float<T>(i < z.latent ? low[i] * scale * latent_weight[i] : rotated_at(low + z.latent, i - z.latent));
        }
        at += key_width;
    }
    if (z.has_gate)
        for (int h = threadIdx.x; h < z.heads; h += blockDim.x) gate[(size_t)t * z.heads + h] = 1.0f / (1.0f + expf(-row[at + h]));
}

// One block a token.  Columns of a projected row: q_rank of the query latent, then `latent` of the key/value latent.
template <typename T>
__global__ void latent_norms_kernel(const float* __restrict__ proj, int proj_width, const float* __restrict__ q_weight,
                                    const float* __restrict__ latent_weight, float eps, const int* __restrict__ slots,
                                    T* __restrict__ q_latent, T* __restrict__ cache, int q_rank, int latent) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const float* row = proj + t * proj_width;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sum += row[i] * row[i];
    const float q_scale = rsqrtf(block_sum(sum, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) q_latent[t * q_rank + i] = from_float<T>(row[i] * q_scale * q_weight[i]);
    const int slot = slots ? slots[t] : -1;
    if (slot < 0 || !cache) return;
    const float* low = row + q_rank;
    sum = 0.0f;
    for (int i = threadIdx.x; i < latent; i += blockDim.x) sum += low[i] * low[i];
    const float scale = rsqrtf(block_sum(sum, scratch) / (float)latent + eps);
    T* dst = cache + (size_t)slot * latent;
    for (int i = threadIdx.x; i < latent; i += blockDim.x) dst[i] = from_float<T>(low[i] * scale * latent_weight[i]);
}

template <typename T>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ x, const float* __restrict__ gate, int gate_stride, int tokens, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    for (int t = blockIdx.y; t < tokens; t += gridDim.y) {
        const float g = gate[(size_t)t * gate_stride + c];
        x[(size_t)t * width + c] = from_float<T>(to_float(x[(size_t)t * width + c]) / (1.0f + expf(-g)));
    }
}

}  // namespace

MRS_EXPORT int mrs_add_layernorm(int is_bf16, float* residual, const void* delta, const float* weight, const float* bias, float eps,
                                 void* out, const int* rows, int n_rows, int width, int write_back, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return MRS_BAD_ARGUMENT;
    const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)bias | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && aligned && width <= 4 * LN_CHUNKS * 1024) {
        int threads = ((width + 4 * LN_CHUNKS - 1) / (4 * LN_CHUNKS) + 31) / 32 * 32;
        if (threads < 64) threads = 64;
        if (is_bf16)
            MRS_LAUNCH(add_layernorm_vec_kernel<bf16>, n_rows, threads, 0, stream, residual, (const bf16*)delta, weight, bias, eps,
                       (bf16*)out, rows, width, write_back);
        else
            MRS_LAUNCH(add_layernorm_vec_kernel<float>, n_rows, threads, 0, stream, residual, (const float*)delta, weight, bias, eps,
                       (float*)out, rows, width, write_back);
        MRS_RETURN_LAUNCH_STATUS();
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (is_bf16)
        MRS_LAUNCH(add_layernorm_kernel<bf16>, n_rows, threads, 0, stream, residual, (const bf16*)delta, weight, bias, eps, (bf16*)out,
                   rows, width, write_back);
    else
        MRS_LAUNCH(add_layernorm_kernel<float>, n_rows, threads, 0, stream, residual, (const float*)delta, weight, bias, eps,
                   (float*)out, rows, width, write_back);
    MRS_RETURN_LAUNCH_STATUS();
}

// x *= factor over n float32 elements (logits that a design scales by a constant).
MRS_EXPORT int mrs_scale(float* x, long long n, float factor, void* stream) {
    if (n <= 0) return 0;
    long long blocks = (n + 255) / 256;
    if (blocks > 8LL * mrs_sm_count()) blocks = 8LL * mrs_sm_count();
    MRS_LAUNCH(scale_kernel, (unsigned)blocks, 256, 0, stream, x, n, factor);
    MRS_RETURN_LAUNCH_STATUS();
}

// q_plain [heads, tokens, plain], q_rows [tokens, heads, latent + rotated] (only the rotated columns are written),
// cache rows of latent + rotated elements addressed by `slots` (null or a slot of -1: nothing is kept), gate [tokens, heads].
MRS_EXPORT int mrs_latent_prepare(int is_bf16, const float* proj, int proj_width, const float* latent_weight, float eps,
                                  const float* inv_freq, float magnitude, const int* positions, const int* slots, void* q_plain,
                                  void* q_rows, void* cache, float* gate, int tokens, int heads, int plain, int rotated, int latent,
                                  int rotary, int has_latent, int has_gate, void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || plain <= 0 || rotated < 0 || latent <= 0 || rotary < 0 || rotary > rotated || rotary % 2 || (rotary && !inv_freq) ||
        (has_latent && !latent_weight) || (has_gate && !gate) ||
        proj_width != heads * (plain + rotated) + (has_latent ? latent + rotated : 0) + (has_gate ? heads : 0))
        return MRS_BAD_ARGUMENT;
    LatentSizes z;
    z.heads = heads, z.plain = plain, z.rotated = rotated, z.latent = latent, z.rotary = rotary, z.has_latent = has_latent, z.has_gate = has_gate;
    const size_t smem = (size_t)(rotary > 0 ? rotary : 1) * sizeof(float);
    if (is_bf16)
        MRS_LAUNCH(latent_prepare_kernel<bf16>, tokens, 256, smem, stream, proj, proj_width, latent_weight, eps, inv_freq, magnitude,
                   positions, slots, (bf16*)q_plain, (bf16*)q_rows, (bf16*)cache, gate, tokens, z);
    else
        MRS_LAUNCH(latent_prepare_kernel<float>, tokens, 256, smem, stream, proj, proj_width, latent_weight, eps, inv_freq, magnitude,
                   positions, slots, (float*)q_plain, (float*)q_rows, (float*)cache, gate, tokens, z);
    MRS_RETURN_LAUNCH_STATUS();
}

// q_latent [tokens, q_rank]; cache rows of `latent` elements addressed by `slots` (null or a slot of -1: nothing is kept).
MRS_EXPORT int mrs_latent_norms(int is_bf16, const float* proj, int proj_width, const float* q_weight, const float* latent_weight,
                                float eps, const int* slots, void* q_latent, void* cache, int tokens, int q_rank, int latent,
                                void* stream) {
    if (tokens <= 0) return 0;
    if (q_rank <= 0 || latent <= 0 || proj_width < q_rank + latent || !q_weight || !latent_weight) return MRS_BAD_ARGUMENT;
    if (is_bf16)
        MRS_LAUNCH(latent_norms_kernel<bf16>, tokens, 128, 0, stream, proj, proj_width, q_weight, latent_weight, eps, slots,
                   (bf16*)q_latent, (bf16*)cache, q_rank, latent);
    else
        MRS_LAUNCH(latent_norms_kernel<float>, tokens, 128, 0, stream, proj, proj_width, q_weight, latent_weight, eps, slots,
                   (float*)q_latent, (float*)cache, q_rank, latent);
    MRS_RETURN_LAUNCH_STATUS();
}

// x [tokens, width] of the engine's dtype, in place; gate: float32 rows of gate_stride elements, the columns at `gate`.
MRS_EXPORT int mrs_sigmoid_gate_mul(int is_bf16, void* x, const float* gate, int gate_stride, int tokens, int width, void* stream) {
    if (tokens <= 0 || width <= 0) return 0;
    const int threads = 128;
    const unsigned across = (unsigned)((width + threads - 1) / threads);
    long long down = ((long long)mrs_sm_count() * 16 + across - 1) / across;
    if (down > tokens) down = tokens;
    if (down > 65535) down = 65535;
    if (is_bf16)
        MRS_LAUNCH(sigmoid_gate_mul_kernel<bf16>, dim3(across, (unsigned)down), threads, 0, stream, (bf16*)x, gate, gate_stride, tokens, width);
    else
        MRS_LAUNCH(sigmoid_gate_mul_kernel<float>, dim3(across, (unsigned)down), threads, 0, stream, (float*)x, gate, gate_stride, tokens, width);
    MRS_RETURN_LAUNCH_STATUS();
}
