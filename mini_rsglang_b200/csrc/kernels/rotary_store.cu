// After a fused q | k (| v) (| gate ...) projection with float32 sums: the heads of q and k are rotated by their
// token's position and pass an RMS norm, before or after the rotation; q leaves in the engine's dtype, k goes into
// the key pages, v into the value pages.  What may vary:
//   * rotation: the first `rot` elements of a head turn, pair i being (i, i + rot / 2) or (2 i, 2 i + 1); the
//     pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a), a = position * f_i; cosines and sines come from
//     the step's table [tokens, rot / 2, 2] (float32); rot = 0: no rotation;
//   * the norm x / sqrt(mean(x^2) + eps) over the whole head, with a weight of the head's size (one for all query
//     heads, one for all key heads) or without one; before the rotation, after it, or not at all;
//   * the values: columns of their own, or the key heads as they were projected (before norm and rotation).
// Columns behind q, k and v (gates) are left to whoever reads them.  Key pages [pages, nkv, page, d], value pages
// [pages, nkv, page, e]; slot < 0 writes nothing.  One warp a head; the head waits in shared memory as float32.  Heads of a
// multiple of four elements in rows on 16-byte boundaries (VEC) come and go four elements a lane and access.
#include "common.cuh"

#define ROTARY_MAX_D 256
#define ROTARY_WARPS 8

namespace {

__device__ __forceinline__ void head_norm(float* x, int d, const float* w, float eps, int lane) {
    float sum = 0.0f;
    for (int i = lane; i < d; i += 32) sum += x[i] * x[i];
    const float scale = 1.0f / sqrtf(warp_sum(sum) / (float)d + eps);
    for (int i = lane; i < d; i += 32) x[i] = w ? x[i] * scale * w[i] : x[i] * scale;
    __syncwarp();
}

template <typename T> __device__ __forceinline__ void put4(T* p, float4 v);
template <> __device__ __forceinline__ void put4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void put4<bf16>(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// n elements from float32 `src` to `dst` of the engine's dtype, a warp together
template <typename T, bool VEC>
__device__ __forceinline__ void copy_out(T* dst, const float* src, int n, int lane) {
    if (VEC) {
        for (int i = 4 * lane; i < n; i += 128) put4<T>(dst + i, *reinterpret_cast<const float4*>(src + i));
    } else {
        for (int i = lane; i < n; i += 32) dst[i] = from_float<T>(src[i]);
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(32 * ROTARY_WARPS)
qkv_rotary_store_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ q_norm,
                        const float* __restrict__ k_norm, int norm_mode, float eps, const float* __restrict__ rotations, int rot,
                        int interleaved, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                        const int* __restrict__ slots, int nq, int nkv, int d, int e, int page_size, int values_from_keys) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) float heads[ROTARY_WARPS][ROTARY_MAX_D];
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qw = nq * d, kw = nkv * d;
    const float* row = proj + t * proj_stride;
    const int slot = slots ? slots[t] : -1;
    const bool store = slot >= 0 && k_cache != nullptr;
    const int page = store ? slot / page_size : 0, in_page = store ? slot % page_size : 0;
    const int half = rot / 2;
    const float* turn = rotations ? rotations + t * (size_t)half * 2 : nullptr;
    const int units = nq + nkv + (values_from_keys ? 0 : nkv);
    for (int unit = warp; unit < units; unit += ROTARY_WARPS) {
        if (unit >= nq + nkv) {                              // a value head with columns of its own
            if (!store || !v_cache) continue;
            const int head = unit - nq - nkv;
            const float* src = row + qw + kw + head * e;
            copy_out<T, VEC>(v_cache + (((size_t)page * nkv + head) * page_size + in_page) * e, src, e, lane);
            continue;
        }
        const bool is_q = unit < nq;
        const int head = is_q ? unit : unit - nq;
        if (!is_q && !store) continue;
        const float* src = row + (is_q ? head * d : qw + head * d);
        float* x = heads[warp];
        if (VEC) {
            for (int i = 4 * lane; i < d; i += 128) *reinterpret_cast<float4*>(x + i) = *reinterpret_cast<const float4*>(src + i);
        } else {
            for (int i = lane; i < d; i += 32) x[i] = src[i];
        }
        __syncwarp();
        if (!is_q && values_from_keys && v_cache)            // the value is the key as projected
            copy_out<T, VEC>(v_cache + (((size_t)page * nkv + head) * page_size + in_page) * d, x, d, lane);
        const float* w = is_q ? q_norm : k_norm;
        if (norm_mode == 1) head_norm(x, d, w, eps, lane);
        if (turn) {
            for (int i = lane; i < half; i += 32) {
                const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
                const float c = turn[2 * i], s = turn[2 * i + 1];
                const float u = x[a], v = x[b];
                x[a] = u * c - v * s;
                x[b] = v * c + u * s;
            }
            __syncwarp();
        }
        if (norm_mode == 2) head_norm(x, d, w, eps, lane);
        copy_out<T, VEC>(is_q ? q_out + t * qw + (size_t)head * d : k_cache + (((size_t)page * nkv + head) * page_size + in_page) * d, x, d, lane);
        __syncwarp();
    }
}

// The same for heads of up to 128 elements (a multiple of 4) in rows on 16-byte boundaries, with the head in registers: a
// lane owns four neighbouring elements from the load to the store.  Interleaved pairs lie inside a lane; the partner of a
// split half lies rot / 8 lanes away (rot a multiple of 8), so a rotation is four shuffles; a norm is one sum over the warp.
template <typename T>
__global__ void __launch_bounds__(32 * ROTARY_WARPS)
qkv_rotary_store_regs_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ q_norm,
                             const float* __restrict__ k_norm, int norm_mode, float eps, const float* __restrict__ rotations, int rot,
                             int interleaved, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                             const int* __restrict__ slots, int nq, int nkv, int d, int e, int page_size, int values_from_keys) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qw = nq * d, kw = nkv * d;
    const float* row = proj + t * proj_stride;
    const int slot = slots ? slots[t] : -1;
    const bool store = slot >= 0 && k_cache != nullptr;
    const int page = store ? slot / page_size : 0, in_page = store ? slot % page_size : 0;
    const int half = rot / 2;
    const float* turn = rotations ? rotations + t * (size_t)half * 2 : nullptr;
    const int units = nq + nkv + (values_from_keys ? 0 : nkv);
    const int at = 4 * lane;                                  // this lane's first element of a head
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int unit = warp; unit < units; unit += ROTARY_WARPS) {
        if (unit >= nq + nkv) {                              // a value head with columns of its own
            if (!store || !v_cache) continue;
            const int head = unit - nq - nkv;
            if (at < e) put4<T>(v_cache + (((size_t)page * nkv + head) * page_size + in_page) * e + at,
                                *reinterpret_cast<const float4*>(row + qw + kw + head * e + at));
            continue;
        }
        const bool is_q = unit < nq;
        const int head = is_q ? unit : unit - nq;
        if (!is_q && !store) continue;
        const bool mine = at < d;
        float4 x = mine ? *reinterpret_cast<const float4*>(row + (is_q ? head * d : qw + head * d) + at) : zero;
        if (!is_q && values_from_keys && v_cache && mine)    // the value is the key as projected
            put4<T>(v_cache + (((size_t)page * nkv + head) * page_size + in_page) * d + at, x);
        const float* w = is_q ? q_norm : k_norm;
        const float4 wv = (w && mine && norm_mode) ? *reinterpret_cast<const float4*>(w + at) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if (norm_mode == 1) {
            const float scale = 1.0f / sqrtf(warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w) / (float)d + eps);
            x = make_float4(x.x * scale * wv.x, x.y * scale * wv.y, x.z * scale * wv.z, x.w * scale * wv.w);
        }
        if (turn) {
            if (interleaved) {                               // pairs (at, at + 1) and (at + 2, at + 3): pair numbers at / 2 and at / 2 + 1
                if (at < rot) {
                    const float2 cs = *reinterpret_cast<const float2*>(turn + at);        // pair at / 2: (cos, sin)
                    const float u = x.x, v = x.y;
                    x.x = u * cs.x - v * cs.y, x.y = v * cs.x + u * cs.y;
                }
                if (at + 2 < rot) {
                    const float2 cs = *reinterpret_cast<const float2*>(turn + at + 2);
                    const float u = x.z, v = x.w;
                    x.z = u * cs.x - v * cs.y, x.w = v * cs.x + u * cs.y;
                }
            } else {
                const int away = rot / 8;                    // lanes between an element and its partner
                const bool low = at < half, turns = at < rot;
                const int partner = turns ? (low ? lane + away : lane - away) : lane;
                const float4 other = make_float4(__shfl_sync(0xffffffffu, x.x, partner), __shfl_sync(0xffffffffu, x.y, partner),
                                                 __shfl_sync(0xffffffffu, x.z, partner), __shfl_sync(0xffffffffu, x.w, partner));
                if (turns) {
                    // pair i = (i, i + half): the low element becomes u cos - v sin, the high one v cos + u sin
                    const int i = low ? at : at - half;
                    const float4 c01 = *reinterpret_cast<const float4*>(turn + 2 * i), c23 = *reinterpret_cast<const float4*>(turn + 2 * i + 4);
                    const float sign = low ? -1.0f : 1.0f;
                    x = make_float4(x.x * c01.x + sign * other.x * c01.y, x.y * c01.z + sign * other.y * c01.w,
                                    x.z * c23.x + sign * other.z * c23.y, x.w * c23.z + sign * other.w * c23.w);
                }
            }
        }
        if (norm_mode == 2) {
            const float scale = 1.0f / sqrtf(warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w) / (float)d + eps);
            x = make_float4(x.x * scale * wv.x, x.y * scale * wv.y, x.z * scale * wv.z, x.w * scale * wv.w);
        }
        if (mine)
            put4<T>(is_q ? q_out + t * qw + (size_t)head * d + at : k_cache + (((size_t)page * nkv + head) * page_size + in_page) * d + at, x);
    }
}

}  // namespace

MRS_EXPORT int mrs_qkv_rotary_store(int is_bf16, const float* proj, int proj_stride, const float* q_norm, const float* k_norm,
                                    int norm_mode, float eps, const float* rotations, int rot, int interleaved, void* q_out,
                                    void* k_cache, void* v_cache, const int* slots, int tokens, int nq, int nkv, int d, int e,
                                    int page_size, int values_from_keys, void* s) {
    if (tokens <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || d <= 0 || d > ROTARY_MAX_D || e <= 0 || page_size <= 0 || norm_mode < 0 || norm_mode > 2 || rot < 0 ||
        rot > d || rot % 2 || (rot > 0 && !rotations) || (values_from_keys && e != d) ||
        proj_stride < nq * d + nkv * d + (values_from_keys ? 0 : nkv * e))
        return MRS_BAD_ARGUMENT;
    if (rot == 0) rotations = nullptr;
    const bool vec = d % 4 == 0 && e % 4 == 0 && proj_stride % 4 == 0 &&
                     (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0;
    // heads that fit a warp's registers, four elements a lane: split halves need the partner a whole number of lanes away
    if (vec && d <= 128 && e <= 128 && (rot == 0 || (interleaved ? rot % 2 == 0 : rot % 8 == 0)) && (((uintptr_t)q_norm | (uintptr_t)k_norm) & 15) == 0) {
        if (is_bf16)
            MRS_LAUNCH(qkv_rotary_store_regs_kernel<bf16>, tokens, 32 * ROTARY_WARPS, 0, s, proj, proj_stride, q_norm, k_norm, norm_mode, eps,
                       rotations, rot, interleaved, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, slots, nq, nkv, d, e, page_size, values_from_keys);
        else
            MRS_LAUNCH(qkv_rotary_store_regs_kernel<float>, tokens, 32 * ROTARY_WARPS, 0, s, proj, proj_stride, q_norm, k_norm, norm_mode, eps,
                       rotations, rot, interleaved, (float*)q_out, (float*)k_cache, (float*)v_cache, slots, nq, nkv, d, e, page_size, values_from_keys);
        MRS_RETURN_LAUNCH_STATUS();
    }
#define MRS_ROTARY_STORE(T, VEC)                                                                                                     \
    MRS_LAUNCH((qkv_rotary_store_kernel<T, VEC>), tokens, 32 * ROTARY_WARPS, 0, s, proj, proj_stride, q_norm, k_norm, norm_mode, eps, \
               rotations, rot, interleaved, (T*)q_out, (T*)k_cache, (T*)v_cache, slots, nq, nkv, d, e, page_size, values_from_keys)
    if (is_bf16) {
        if (vec) MRS_ROTARY_STORE(bf16, true); else MRS_ROTARY_STORE(bf16, false);
    } else {
        if (vec) MRS_ROTARY_STORE(float, true); else MRS_ROTARY_STORE(float, false);
    }
#undef MRS_ROTARY_STORE
    MRS_RETURN_LAUNCH_STATUS();
}
