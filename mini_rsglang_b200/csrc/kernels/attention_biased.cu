// Paged causal grouped-query attention with the extras that some designs put around the scores:
//   score = (q . k) * scale;  score <- cap * tanh(score / cap)  (cap > 0);
//   score += bias[min(i - j, bias_rows - 1), head]              (a table by distance, float32);
//   key j is seen by query i when j <= i and (i - j < window or j < keep_first)   (window 0: every key);
//   or, with chunk > 0 (and no window), when j <= i and floor(j / chunk) = floor(i / chunk): chunks counted from position 0;
//   softmax with a sink: p_j = exp(s_j) / (exp(z) + sum exp(s_j))   (sink != 0; z = sink_logits[head], or 0 without a table:
//   one more term in the denominator that has no key and no value and is not scaled), else the usual one;
//   out = (sum p_j v_j) * gate[token, head]                     (gate float32, may be null).
// Keys have d elements a head and values e (the two need not agree).  Scores, softmax and sums are float32.
// Without value pages the values are the first e elements of the key rows (a latent that serves as key and as
// value: the cache holds one row a token).  A key on a page that was given back (-1 in the table) counts as unseen.
// This is the CUDA-core version: float32 or bfloat16 storage, keys of up to 1,152 and values of up to 1,024 elements; it is
// the attention of the 32-bit path and the device-side reference of the tensor-core version.
//
// One warp per (token, query head).  The keys a query sees are up to two runs of positions, the kept first
// ones and the window; the warp walks them as one list, 32 at a time: lane j scores key j with a full dot
// product, the warp reduces once per tile (online softmax), then all lanes add the 32 weighted value rows.
#include "common.cuh"

#define ATTN_MAX_D 1152
#define ATTN_MAX_E 1024
#define ATTN_WARPS 4

template <typename T, int EREGS>
__global__ void attention_biased_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                             const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                             const int* __restrict__ block_table, const float* __restrict__ bias,
                                             const float* __restrict__ gate, T* __restrict__ out, int tokens, int nq, int nkv,
                                             int d, int e, int page_size, int table_width, float scale, float cap, int window,
                                             int keep_first, int bias_rows, int sink, const float* __restrict__ sink_logits, int chunk) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float q_s[ATTN_WARPS][ATTN_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * ATTN_WARPS + warp;
    if (unit >= (long long)tokens * nq) return;
    const int t = (int)(unit / nq), h = (int)(unit % nq);
    const int g = h / (nq / nkv);
    const int pos = positions[t];
    const int length = pos + 1;
    // first position of the window, or of the query's chunk
    const int first = chunk > 0 ? (pos / chunk) * chunk : (window > 0 ? max(0, length - window) : 0);
    const int kept = chunk > 0 ? 0 : min(keep_first, first);        // positions [0, kept) lie before a window and stay seen
    const int seen = kept + (length - first);
    const int* pages = block_table + (size_t)seq_of_token[t] * table_width;
    const T* q_row = q + ((size_t)t * nq + h) * d;
    for (int x = lane; x < d; x += 32) q_s[warp][x] = to_float(q_row[x]);
    __syncwarp();

    const int v_stride = v_cache ? e : d;             // no value pages: a value is the head of its key row
    const T* values = v_cache ? v_cache : k_cache;
    float acc[EREGS];
#pragma unroll
    for (int i = 0; i < EREGS; ++i) acc[i] = 0.0f;
    float running_max = sink ? (sink_logits ? sink_logits[h] : 0.0f) : -CUDART_INF_F, running_sum = sink ? 1.0f : 0.0f;

    for (int base = 0; base < seen; base += 32) {
        const int u = base + lane;
        const int p = u < kept ? u : first + (u - kept);
        float score = -CUDART_INF_F;
        const int page = u < seen ? pages[p / page_size] : -1;
        if (page >= 0) {
            const T* k_row = k_cache + (((size_t)page * nkv + g) * page_size + (p % page_size)) * d;
            float dot = 0.0f;
            for (int x = 0; x < d; ++x) dot += q_s[warp][x] * to_float(k_row[x]);
            score = dot * scale;
            if (cap > 0.0f) score = cap * tanhf(score / cap);
            if (bias) score += bias[(size_t)min(pos - p, bias_rows - 1) * nq + h];
        }
        const float new_max = fmaxf(running_max, warp_max(score));
        const float alpha = new_max == -CUDART_INF_F ? 1.0f : expf(running_max - new_max);
        const float prob = page >= 0 ? expf(score - new_max) : 0.0f;
        running_sum = running_sum * alpha + warp_sum(prob);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < EREGS; ++i) acc[i] *= alpha;
        const int in_tile = min(32, seen - base);
        for (int j = 0; j < in_tile; ++j) {
            const float pj = __shfl_sync(0xffffffffu, prob, j);
            const int uj = base + j;
            const int pj_pos = uj < kept ? uj : first + (uj - kept);
            const int page = pages[pj_pos / page_size];
            if (page < 0) continue;
            const T* v_row = values + (((size_t)page * nkv + g) * page_size + (pj_pos % page_size)) * v_stride;
#pragma unroll
            for (int i = 0; i < EREGS; ++i) {
                const int x = lane + 32 * i;
                if (x < e) acc[i] += pj * to_float(v_row[x]);
            }
        }
    }
    T* o = out + ((size_t)t * nq + h) * e;
    const float factor = (running_sum > 0.0f ? 1.0f / running_sum : 0.0f) * (gate ? gate[(size_t)t * nq + h] : 1.0f);
#pragma unroll
    for (int i = 0; i < EREGS; ++i) {
        const int x = lane + 32 * i;
        if (x < e) o[x] = from_float<T>(acc[i] * factor);
    }
}

MRS_EXPORT int mrs_attention_biased_simt(int is_bf16, const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                         const int* seq_of_token, const int* block_table, const float* bias, const float* gate,
                                         void* out, int tokens, int nq, int nkv, int d, int e, int page_size, int table_width,
                                         float scale, float cap, int window, int keep_first, int bias_rows, int sink,
                                         const float* sink_logits, int chunk, void* stream) {
    if (tokens <= 0) return 0;
    if (d <= 0 || d > ATTN_MAX_D || e <= 0 || e > ATTN_MAX_E || (!v_cache && e > d) || nkv <= 0 || nq % nkv || (bias && bias_rows <= 0) || window < 0 ||
        keep_first < 0 || chunk < 0 || (chunk > 0 && window > 0) || (sink_logits && !sink))
        return MRS_BAD_ARGUMENT;
    const long long units = (long long)tokens * nq;
    const unsigned blocks = (unsigned)((units + ATTN_WARPS - 1) / ATTN_WARPS);
#define MRS_BIASED_SIMT(T, EREGS)                                                                                              \
    MRS_LAUNCH((attention_biased_simt_kernel<T, EREGS>), blocks, 32 * ATTN_WARPS, 0, stream, (const T*)q, (const T*)k_cache,      \
               (const T*)v_cache, positions, seq_of_token, block_table, bias, gate, (T*)out, tokens, nq, nkv, d, e, page_size,    \
               table_width, scale, cap, window, keep_first, bias_rows, sink, sink_logits, chunk)
    if (is_bf16) {
        if (e <= 128) MRS_BIASED_SIMT(bf16, 4); else if (e <= 256) MRS_BIASED_SIMT(bf16, 8); else if (e <= 512) MRS_BIASED_SIMT(bf16, 16); else MRS_BIASED_SIMT(bf16, 32);
    } else {
        if (e <= 128) MRS_BIASED_SIMT(float, 4); else if (e <= 256) MRS_BIASED_SIMT(float, 8); else if (e <= 512) MRS_BIASED_SIMT(float, 16); else MRS_BIASED_SIMT(float, 32);
    }
#undef MRS_BIASED_SIMT
    MRS_RETURN_LAUNCH_STATUS();
}
