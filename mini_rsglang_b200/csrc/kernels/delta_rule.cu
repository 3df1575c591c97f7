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
//   delta_scan        the recurrence token by token; one block a (sequence, head, slice of S's columns)
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

// Thread (column c of the block's slice, part p): rows p * PER .. p * PER + PER - 1 of column c of S in registers; the
// lanes of one column are neighbours, so that the two sums over d are a few shuffles.  The next token's inputs are
// asked for before this token's arithmetic.
template <int PER>
__global__ void delta_scan_kernel(const float* __restrict__ qkv, int qkv_width, const float* __restrict__ coef,
                                  float* __restrict__ state, long long state_stride, const int* __restrict__ positions,
                                  const int* __restrict__ q_start, const int* __restrict__ state_slots, float* __restrict__ out,
                                  int heads, int groups, int d, int e, int parts, int cols, int write_state) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int first = q_start[seq], last = q_start[seq + 1];
    const int slot = state_slots[seq];
    if (slot < 0 || last <= first) return;
    const int part = threadIdx.x % parts, col = blockIdx.z * cols + threadIdx.x / parts;
    const bool live = col < e;                       // a slice may overhang the head; its threads still take part in the shuffles
    const int c = live ? col : 0;
    const int group = head / (heads / groups);
    const int row0 = part * PER;
    float* mine = state + (long long)slot * state_stride + ((size_t)head * d) * e + c;
    float s[PER];
    const bool fresh = positions[first] == 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) s[i] = (!fresh && live && row0 + i < d) ? mine[(size_t)(row0 + i) * e] : 0.0f;

    const size_t q_at = (size_t)group * d + row0, k_at = (size_t)(groups + group) * d + row0, v_at = (size_t)2 * groups * d + (size_t)head * e + c;
    float kq[2][2][PER], v[2], beta[2], decay[2];
    auto fetch = [&](int t, int b) {
        const float* row = qkv + (size_t)t * qkv_width;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            kq[b][0][i] = row0 + i < d ? row[k_at + i] : 0.0f;
            kq[b][1][i] = row0 + i < d ? row[q_at + i] : 0.0f;
        }
        v[b] = row[v_at];
        beta[b] = coef[(size_t)t * 2 * heads + head];
        decay[b] = coef[(size_t)t * 2 * heads + heads + head];
    };
    fetch(first, 0);
    for (int t = first; t < last; ++t) {
        const int b = (t - first) & 1;
        if (t + 1 < last) fetch(t + 1, b ^ 1);
        float r = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            s[i] *= decay[b];
            r += s[i] * kq[b][0][i];
        }
        for (int o = parts >> 1; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        const float u = beta[b] * (v[b] - r);
        float y = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            s[i] += kq[b][0][i] * u;
            y += s[i] * kq[b][1][i];
        }
        for (int o = parts >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (live && part == 0) out[(size_t)t * heads * e + (size_t)head * e + c] = y;
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
    constexpr int PER = 16;
    int parts = 1;
    while (parts * PER < d) parts <<= 1;                 // lanes a column: a power of two, at most 32
    // columns a block: as few as still give every multiprocessor two blocks, at least a warp's worth of threads
    int cols = 128 / parts;
    const long long pairs = (long long)sequences * heads;
    while (cols * parts > 32 && pairs * ((e + cols - 1) / cols) < 2LL * mrs_sm_count()) cols >>= 1;
    const int slices = (e + cols - 1) / cols;
    if (slices > 65535) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(delta_scan_kernel<PER>, dim3(sequences, heads, slices), cols * parts, 0, stream, qkv, 2 * groups * d + heads * e, coef,
               state, state_stride, positions, q_start, state_slots, out, heads, groups, d, e, parts, cols, write_state);
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
