// What enters the float32 residual stream besides a plain table row, and what re-enters it:
//
//   embed_pairs   stream[t] = table[id] * scale + pair_table[row], row = (previous id * mul_prev + id * mul_cur) mod
//                 buckets, and row number `buckets` (the table's last) for the first token of a sequence.  The token
//                 before the first one of a step's portion is the request's state: `last_token` [slots] int32 holds
//                 the last token that every request brought; the thread of a sequence's first row reads it and then
//                 (unless told to write nothing) puts the portion's last token there, so nothing else touches it.
//   concat_rows   out[t] = [a[t] ; b[t]] in the engine's dtype, a and b float32 [rows, width]: the operand of a
//                 product over the stream beside another stream-sized tensor.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embed_pairs_kernel(const T* __restrict__ table, const T* __restrict__ pair_table, const int* __restrict__ ids,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ q_start, const int* __restrict__ state_slots, int* __restrict__ last_token,
                                   float* __restrict__ stream, int width, int vocab, float scale, int buckets, long long mul_prev,
                                   long long mul_cur, int write_state) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;          // a token that a sampler has not filled in yet never reaches here; stay in the table
    const int seq = seq_of_token[t];
    const int first = q_start[seq], end = q_start[seq + 1];
    const int slot = state_slots[seq];
    int row = buckets;
    if (positions[t] > 0) {
        int previous = 0;
        if (t > first && t < end) previous = ids[t - 1];
        else if (slot >= 0) previous = last_token[slot];
        long long r = ((long long)previous * mul_prev + (long long)id * mul_cur) % buckets;
        if (r < 0) r += buckets;
        row = (int)r;
    }
    __syncthreads();                             // every thread has read the state before one of them writes it
    if (threadIdx.x == 0 && write_state && t == first && end > first && slot >= 0) last_token[slot] = ids[end - 1];
    const T* a = table + (size_t)id * width;
    const T* b = pair_table + (size_t)row * width;
    float* o = stream + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_float(a[i]) * scale + to_float(b[i]);
}

template <typename T>
__global__ void concat_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int rows, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long long n = (long long)rows * 2 * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / (2 * width);
        const int c = (int)(i % (2 * width));
        out[i] = from_float<T>(c < width ? a[r * width + c] : b[r * width + c - width]);
    }
}

// The same, four elements a thread and step: width a multiple of 4, all three on 16-byte boundaries.
template <typename T>
__global__ void concat_rows_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, T* __restrict__ out, int rows, int quads) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;       // a quad of the joined row
    if (c >= 2 * quads) return;
    const float4* src = c < quads ? a + c : b + (c - quads);
    for (int r = blockIdx.y; r < rows; r += gridDim.y) {
        const float4 v = src[(size_t)r * quads];
        T* o = out + ((size_t)r * 2 * quads + c) * 4;
        if (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(o) = v;
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 raw;
            raw.x = *reinterpret_cast<uint32_t*>(&lo);
            raw.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(o) = raw;
        }
    }
}

}  // namespace

MRS_EXPORT int mrs_embed_pairs(int is_bf16, const void* table, const void* pair_table, const int* ids, const int* positions,
                               const int* seq_of_token, const int* q_start, const int* state_slots, int* last_token, float* stream,
                               int tokens, int width, int vocab, float scale, int buckets, long long mul_prev, long long mul_cur,
                               int write_state, void* s) {
    if (tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0 || buckets <= 0 || !last_token) return MRS_BAD_ARGUMENT;
    const int threads = width >= 1024 ? 256 : 128;
    if (is_bf16)
        MRS_LAUNCH(embed_pairs_kernel<bf16>, tokens, threads, 0, s, (const bf16*)table, (const bf16*)pair_table, ids, positions,
                   seq_of_token, q_start, state_slots, last_token, stream, width, vocab, scale, buckets, mul_prev, mul_cur, write_state);
    else
        MRS_LAUNCH(embed_pairs_kernel<float>, tokens, threads, 0, s, (const float*)table, (const float*)pair_table, ids, positions,
                   seq_of_token, q_start, state_slots, last_token, stream, width, vocab, scale, buckets, mul_prev, mul_cur, write_state);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_concat_rows(int is_bf16, const float* a, const float* b, void* out, int rows, int width, void* s) {
    if (rows <= 0) return 0;
    if (width <= 0) return MRS_BAD_ARGUMENT;
    if (width % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0) {
        const int quads = width / 4;
        const unsigned across = (unsigned)((2 * quads + 127) / 128);
        long long down = ((long long)mrs_sm_count() * 16 + across - 1) / across;
        if (down > rows) down = rows;
        if (down > 65535) down = 65535;
        if (is_bf16)
            MRS_LAUNCH(concat_rows_vec_kernel<bf16>, dim3(across, (unsigned)down), 128, 0, s, (const float4*)a, (const float4*)b, (bf16*)out, rows, quads);
        else
            MRS_LAUNCH(concat_rows_vec_kernel<float>, dim3(across, (unsigned)down), 128, 0, s, (const float4*)a, (const float4*)b, (float*)out, rows, quads);
        MRS_RETURN_LAUNCH_STATUS();
    }
    long long blocks = ((long long)rows * 2 * width + 255) / 256;
    if (blocks > 16LL * mrs_sm_count()) blocks = 16LL * mrs_sm_count();
    if (is_bf16)
        MRS_LAUNCH(concat_rows_kernel<bf16>, (unsigned)blocks, 256, 0, s, a, b, (bf16*)out, rows, width);
    else
        MRS_LAUNCH(concat_rows_kernel<float>, (unsigned)blocks, 256, 0, s, a, b, (float*)out, rows, width);
    MRS_RETURN_LAUNCH_STATUS();
}
