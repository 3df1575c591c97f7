// The gated delta rule: a recurrence whose state is a matrix S [d, e] per (request, head) that forgets by a scalar a
// token and then corrects what it holds under the token's key towards the token's value:
//
//     S <- g_t S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t
//
// with q_t, k_t [d] (shared by the query heads of a group) made unit vectors, x / sqrt(sum x^2 + unit_eps), q also times
// a constant; beta_t = sigmoid(b_t); g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias_h)).  Afterwards every head's o_t is
// divided by its root mean square, multiplied by a weight and by silu of a gate.
//
// Everything here is float32: unit norms, step sizes, decays, the state and the read-out.  S lives in the request's
// state slot between steps [slots, heads, d, e]; where a sequence starts at position 0 its state counts as zero, whatever
// the slot held (slots are used again).  State slot -1: a padding sequence, nothing is read or written.  The step's
// facts come from device arrays only, so a step can be recorded.
//
//   delta_prepare     per token: q and k of every group to unit length in place; beta and g of every head
//   delta_scan        the recurrence token by token; one block a (sequence, head, slice of S's columns), the tokens'
//                     inputs staged through shared memory ahead of their use
//   head_norm_gate    o / rms(o) * weight * silu(gate) per (token, head)
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

// qkv [tokens, 2 * groups * d + heads * e] float32: q of every group, k of every group, v of every head.
// raw [tokens, raw_stride] float32: at column b_offset one b a head, at a_offset one a a head.
// coef [tokens, 2 * heads]: beta, then g.
__global__ void delta_prepare_kernel(float* __restrict__ qkv, int qkv_width, const float* __restrict__ raw, int raw_stride,
                                     int b_offset, int a_offset, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     float* __restrict__ coef, int groups, int d, int heads, float unit_eps, float q_factor) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* row = qkv + t * qkv_width;
    for (int unit = warp; unit < 2 * groups; unit += warps) {          // units 0 .. groups - 1: q; the rest: k
        float* x = row + (size_t)unit * d;
        float sum = 0.0f;
        for (int i = lane; i < d; i += 32) sum += x[i] * x[i];
        const float factor = (unit < groups ? q_factor : 1.0f) / sqrtf(warp_sum(sum) + unit_eps);
        for (int i = lane; i < d; i += 32) x[i] *= factor;
    }
    const float* r = raw + t * raw_stride;
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        coef[t * 2 * heads + h] = 1.0f / (1.0f + expf(-r[b_offset + h]));
        coef[t * 2 * heads + heads + h] = expf(-expf(a_log[h]) * softplus_f(r[a_offset + h] + dt_bias[h]));
    }
}

__device__ __forceinline__ uint32_t shared_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void copy_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(shared_address(dst)), "l"(src));
}
__device__ __forceinline__ void copy_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(shared_address(dst)), "l"(src));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Thread (column c of the block's slice, part p): rows p * PER .. p * PER + PER - 1 of column c of S in registers (PER is
// 16 or 8, the launcher's choice); the
// PARTS lanes of one column are neighbours, so that the two sums over d are log2(PARTS) shuffles.  The tokens' inputs (k and
// q of the head's group, the slice of v, beta and g) come in batches of `batch_tokens` through two stages of shared memory:
// the next batch is copied while this one is computed, and the threads of a block share what they read.  A token in shared
// memory: k [PARTS * PITCH] | q [PARTS * PITCH] | v [cols rounded up to 4] | beta, g, 0, 0, with PITCH = PER + 4, so that
// the 16-byte reads of the parts fall on different banks; the rows beyond d stay zero.
//
// One warp a scheduler is all that a single sequence offers, so every instruction's latency shows.  What a thread copies is
// therefore the same in every batch and worked out once, ahead of the loop (`Copies`); and the chain from token to token is
// only: the sum over S's old rows times k, the shuffles, u, one fused multiply-add a row.  The decay is applied to S beside
// the shuffles (r = g * sum(S_old k)), and the read-out of one token overlaps the next one's chain.
template <int N>
struct Copies {
    int src[N], dst[N], token[N];      // offsets in floats from the batch's first row and from the stage; a huge token: none
};

template <int PER, int PARTS>
__global__ void __launch_bounds__(128) delta_scan_kernel(const float* __restrict__ qkv, int qkv_width, const float* __restrict__ coef,
                                  float* __restrict__ state, long long state_stride, const int* __restrict__ positions,
                                  const int* __restrict__ q_start, const int* __restrict__ state_slots, float* __restrict__ out,
                                  int heads, int groups, int d, int e, int cols, int batch_tokens, int wide_copies,
                                  int write_state) {
    extern __shared__ __align__(16) float stage[];
    constexpr int PITCH = PER + 4, ROWS = PARTS * PITCH;
    constexpr int WIDE = 8, NARROW = 3;                    // copies a thread and batch that are worked out ahead
    pdl_launch_dependents();
    const int cols_pad = (cols + 3) & ~3;
    const int token_floats = 2 * ROWS + cols_pad + 4, stage_floats = batch_tokens * token_floats;
    for (int i = threadIdx.x; i < 2 * stage_floats; i += blockDim.x) stage[i] = 0.0f;
    __syncthreads();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int first = q_start[seq], last = q_start[seq + 1];
    const int slot = state_slots[seq];
    if (slot < 0 || last <= first) return;
    const int part = threadIdx.x % PARTS, col_in_slice = threadIdx.x / PARTS, col = blockIdx.z * cols + col_in_slice;
    const bool live = col < e;                       // a slice may overhang the head; its threads still take part in the shuffles
    const int c = live ? col : 0;
    const int group = head / (heads / groups);
    const int row0 = part * PER;
    float* mine = state + (long long)slot * state_stride + ((size_t)head * d) * e + c;
    float s[PER];
    const bool fresh = positions[first] == 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) s[i] = (!fresh && live && row0 + i < d) ? mine[(size_t)(row0 + i) * e] : 0.0f;

    const int q_at = group * d, k_at = (groups + group) * d, v_at = 2 * groups * d + head * e + (int)blockIdx.z * cols;
    const int live_cols = min(cols, e - (int)blockIdx.z * cols);
    // copy number i of a batch's keys and queries: token j, k or q, elements el .. of the vector
    const int width = wide_copies ? d >> 2 : d, vector_copies = batch_tokens * 2 * width;
    auto vector_copy = [&](int i, int& src, int& dst) {
        const int j = i / (2 * width), r = i % (2 * width), which = r / width, el = (r % width) * (wide_copies ? 4 : 1);
        src = j * qkv_width + (which ? q_at : k_at) + el;
        dst = j * token_floats + which * ROWS + (el / PER) * PITCH + el % PER;
        return j;
    };
    // copy number i of a batch's values and coefficients: token j, a column of v, beta or g
    const int scalar_copies = batch_tokens * (live_cols + 2);
    auto scalar_copy = [&](int i, long long& src, int& dst) {
        const int j = i / (live_cols + 2), r = i % (live_cols + 2);
        if (r < live_cols) {
            src = (long long)j * qkv_width + v_at + r;
            dst = j * token_floats + 2 * ROWS + r;
        } else {
            src = -1 - ((long long)j * 2 * heads + (r == live_cols ? head : heads + head));      // below zero: from coef
            dst = j * token_floats + 2 * ROWS + cols_pad + (r - live_cols);
        }
        return j;
    };
    Copies<WIDE> wide;
    Copies<NARROW> narrow;
    long long narrow_src[NARROW];
    const int longest = min(batch_tokens, last - first);       // a decoded token alone needs the first token's copies only
#pragma unroll
    for (int i = 0; i < WIDE; ++i) {
        const int at = threadIdx.x + i * blockDim.x;
        wide.token[i] = at < longest * 2 * width ? vector_copy(at, wide.src[i], wide.dst[i]) : (1 << 30);
    }
#pragma unroll
    for (int i = 0; i < NARROW; ++i) {
        const int at = threadIdx.x + i * blockDim.x;
        narrow.token[i] = at < longest * (live_cols + 2) ? scalar_copy(at, narrow_src[i], narrow.dst[i]) : (1 << 30);
    }
    auto issue = [&](int t0, int n, int buffer) {
        float* base = stage + buffer * stage_floats;
        const float* rows = qkv + (size_t)t0 * qkv_width;
        const float* facts = coef + (size_t)t0 * 2 * heads;
#pragma unroll
        for (int i = 0; i < WIDE; ++i)
            if (wide.token[i] < n) {
                if (wide_copies) copy_async16(base + wide.dst[i], rows + wide.src[i]);
                else copy_async4(base + wide.dst[i], rows + wide.src[i]);
            }
        for (int at = threadIdx.x + WIDE * blockDim.x; at < vector_copies; at += blockDim.x) {      // sizes beyond the usual
            int src, dst;
            if (vector_copy(at, src, dst) < n) {
                if (wide_copies) copy_async16(base + dst, rows + src);
                else copy_async4(base + dst, rows + src);
            }
        }
#pragma unroll
        for (int i = 0; i < NARROW; ++i)
            if (narrow.token[i] < n) copy_async4(base + narrow.dst[i], narrow_src[i] >= 0 ? rows + narrow_src[i] : facts + (-1 - narrow_src[i]));
        for (int at = threadIdx.x + NARROW * blockDim.x; at < scalar_copies; at += blockDim.x) {
            long long src;
            int dst;
            if (scalar_copy(at, src, dst) < n) copy_async4(base + dst, src >= 0 ? rows + src : facts + (-1 - src));
        }
        copy_async_commit();
    };
    const int batches = (last - first + batch_tokens - 1) / batch_tokens;
    const int token_tail = 2 * ROWS + cols_pad;
    float* out_at = out + (size_t)first * heads * e + (size_t)head * e + c;
    const size_t out_step = (size_t)heads * e;
    const bool writes = live && part == 0;
    issue(first, min(batch_tokens, last - first), 0);
    for (int b = 0; b < batches; ++b) {
        const int t0 = first + b * batch_tokens, n = min(batch_tokens, last - t0);
        if (b + 1 < batches) {
            issue(t0 + batch_tokens, min(batch_tokens, last - t0 - batch_tokens), (b + 1) & 1);
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncthreads();
        const float* token = stage + (b & 1) * stage_floats + part * PITCH;
#pragma unroll 2
        for (int j = 0; j < n; ++j, token += token_floats, out_at += out_step) {
            float k[PER], q[PER];
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const float4 kk = *reinterpret_cast<const float4*>(token + i);
                const float4 qq = *reinterpret_cast<const float4*>(token + ROWS + i);
                k[i] = kk.x, k[i + 1] = kk.y, k[i + 2] = kk.z, k[i + 3] = kk.w;
                q[i] = qq.x, q[i + 1] = qq.y, q[i + 2] = qq.z, q[i + 3] = qq.w;
            }
            const float* tail = token - part * PITCH + token_tail;
            const float v = (tail - cols_pad)[col_in_slice], beta = tail[0], decay = tail[1];
            float r4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < PER; ++i) r4[i & 3] = fmaf(s[i], k[i], r4[i & 3]);
            float r = (r4[0] + r4[1]) + (r4[2] + r4[3]);
#pragma unroll
            for (int o = PARTS >> 1; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
#pragma unroll
            for (int i = 0; i < PER; ++i) s[i] *= decay;                 // beside the shuffles, off the chain
            const float u = beta * (v - decay * r);
            float y4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                s[i] = fmaf(k[i], u, s[i]);
                y4[i & 3] = fmaf(s[i], q[i], y4[i & 3]);
            }
            float y = (y4[0] + y4[1]) + (y4[2] + y4[3]);
#pragma unroll
            for (int o = PARTS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (writes) *out_at = y;
        }
        __syncthreads();                                  // the stage is copied into again two batches on
    }
    if (write_state && live) {
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (row0 + i < d) mine[(size_t)(row0 + i) * e] = s[i];
    }
}

// One warp a (token, head): out = o / sqrt(mean(o^2) + eps) * weight * silu(gate).  o [tokens, heads * e] float32; gate a
// column range of wider float32 rows; weight [e], shared by the heads.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride,
                                      const float* __restrict__ weight, float eps, T* __restrict__ out, int tokens, int heads, int e) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)tokens * heads) return;
    const size_t t = (size_t)(unit / heads);
    const int h = (int)(unit % heads);
    const float* x = o + t * heads * e + (size_t)h * e;
    const float* g = gate + t * gate_stride + (size_t)h * e;
    float sum = 0.0f;
    for (int i = lane; i < e; i += 32) sum += x[i] * x[i];
    const float scale = 1.0f / sqrtf(warp_sum(sum) / (float)e + eps);
    T* dst = out + t * heads * e + (size_t)h * e;
    for (int i = lane; i < e; i += 32) dst[i] = from_float<T>(x[i] * scale * weight[i] * (g[i] / (1.0f + expf(-g[i]))));
}

}  // namespace

MRS_EXPORT int mrs_delta_prepare(float* qkv, const float* raw, int raw_stride, int b_offset, int a_offset, const float* a_log,
                                 const float* dt_bias, float* coef, int tokens, int groups, int d, int heads, int e, float unit_eps,
                                 float q_factor, void* stream) {
    if (tokens <= 0) return 0;
    if (groups <= 0 || d <= 0 || heads <= 0 || e <= 0 || heads % groups) return MRS_BAD_ARGUMENT;
    const int units = 2 * groups;
    const int threads = units >= 8 ? 256 : (units >= 4 ? 128 : 64);
    MRS_LAUNCH(delta_prepare_kernel, tokens, threads, 0, stream, qkv, 2 * groups * d + heads * e, raw, raw_stride, b_offset, a_offset,
               a_log, dt_bias, coef, groups, d, heads, unit_eps, q_factor);
    MRS_RETURN_LAUNCH_STATUS();
}

// state [slots, heads, d, e] float32 with `state_stride` floats from slot to slot; out [tokens, heads * e] float32.
MRS_EXPORT int mrs_delta_scan(const float* qkv, const float* coef, float* state, long long state_stride, const int* positions,
                              const int* q_start, const int* state_slots, float* out, int tokens, int sequences, int heads,
                              int groups, int d, int e, int write_state, void* stream) {
    if (tokens <= 0 || sequences <= 0) return 0;
    if (groups <= 0 || d <= 0 || d > 512 || heads <= 0 || e <= 0 || heads % groups || heads > 65535) return MRS_BAD_ARGUMENT;
    const long long pairs = (long long)sequences * heads;
    int per, parts, cols, slices;
    auto plan = [&](int rows) {
        per = rows;
        parts = 1;
        while (parts * per < d) parts <<= 1;             // lanes a column: a power of two, at most 32
        // columns a block: four warps' worth of threads (they share the tokens' keys and queries in shared memory), fewer
        // while the blocks would leave half the multiprocessors idle, at least a warp's worth of threads
        cols = 128 / parts;
        while (cols > e && cols * parts > 32) cols >>= 1;
        while (cols * parts > 32 && pairs * ((e + cols - 1) / cols) * 2 < mrs_sm_count()) cols >>= 1;
        slices = (e + cols - 1) / cols;
    };
    // rows of a column a thread: 16; 8 where long portions come as more blocks than multiprocessors, so that more of them
    // are resident side by side (measured: from 1.1 to 1.3 times as fast there, slower for short portions and few blocks)
    plan(16);
    if (d <= 256 && tokens >= 256LL * sequences && pairs * slices > mrs_sm_count()) plan(8);
    if (slices > 65535) return MRS_BAD_ARGUMENT;
    const int qkv_width = 2 * groups * d + heads * e;
    const int token_floats = 2 * parts * (per + 4) + ((cols + 3) & ~3) + 4;
    int batch_tokens = (48 * 1024) / (2 * token_floats * (int)sizeof(float));
    if (batch_tokens > 8) batch_tokens = 8;
    if (batch_tokens < 1) return MRS_BAD_ARGUMENT;
    const int wide_copies = d % 4 == 0 && qkv_width % 4 == 0 && ((uintptr_t)qkv & 15) == 0;
    const dim3 grid(sequences, heads, slices);
    const size_t shared = 2 * (size_t)batch_tokens * token_floats * sizeof(float);
#define MRS_DELTA_SCAN(PER, PARTS)                                                                                                   \
    MRS_LAUNCH((delta_scan_kernel<PER, PARTS>), grid, cols * PARTS, shared, stream, qkv, qkv_width, coef, state, state_stride,       \
               positions, q_start, state_slots, out, heads, groups, d, e, cols, batch_tokens, wide_copies, write_state)
#define MRS_DELTA_SCAN_ROWS(PER)                                                                                                     \
    switch (parts) {                                                                                                                 \
        case 1: MRS_DELTA_SCAN(PER, 1); break;                                                                                       \
        case 2: MRS_DELTA_SCAN(PER, 2); break;                                                                                       \
        case 4: MRS_DELTA_SCAN(PER, 4); break;                                                                                       \
        case 8: MRS_DELTA_SCAN(PER, 8); break;                                                                                       \
        case 16: MRS_DELTA_SCAN(PER, 16); break;                                                                                     \
        default: MRS_DELTA_SCAN(PER, 32); break;                                                                                     \
    }
    if (per == 16) { MRS_DELTA_SCAN_ROWS(16) } else { MRS_DELTA_SCAN_ROWS(8) }
#undef MRS_DELTA_SCAN_ROWS
#undef MRS_DELTA_SCAN
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_head_norm_gate(int is_bf16, const float* o, const float* gate, int gate_stride, const float* weight, float eps,
                                  void* out, int tokens, int heads, int e, void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || e <= 0) return MRS_BAD_ARGUMENT;
    const int warps = 4;
    const long long units = (long long)tokens * heads;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    if (is_bf16)
        MRS_LAUNCH(head_norm_gate_kernel<bf16>, blocks, 32 * warps, 0, stream, o, gate, gate_stride, weight, eps, (bf16*)out, tokens, heads, e);
    else
        MRS_LAUNCH(head_norm_gate_kernel<float>, blocks, 32 * warps, 0, stream, o, gate, gate_stride, weight, eps, (float*)out, tokens, heads, e);
    MRS_RETURN_LAUNCH_STATUS();
}
