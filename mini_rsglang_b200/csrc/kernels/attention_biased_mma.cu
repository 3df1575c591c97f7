// The biased, windowed attention (see attention_biased.cu for the formulas) on the tensor cores: bfloat16 in,
// float32 scores, softmax and sums; compiled for one pair of head sizes, -DMRS_HEAD_DIM=<keys> -DMRS_VALUE_DIM=<values>,
// both multiples of 16, values up to 256.  With -DMRS_VALUES_IN_KEYS=1 there are no value pages: a value is the first
// MRS_VALUE_DIM elements of its key row (a latent that serves as key and as value), a block of rows is fetched once and
// read by both products, and key rows may have up to 640 elements.
//
// As in attention_mma.cu a *tile* is a run of consecutive tokens of one request whose query rows are the pairs
// (token, head within the group), so a key is read once for the whole group of query heads:
//   rows mode (64 rows, 4 warps x 16 rows): prompt portions; every warp walks all key blocks of the tile;
//   keys mode (16 rows shared by 4 warps):  decoded tokens and short portions; warp w takes keys 16w .. 16w + 15
//                                           of every block of 64 and the four partial results are merged.
// The keys a tile sees are two runs of blocks, those that hold kept first positions and those of the window; the
// blocks between them are skipped, and what a single row sees is decided score by score.  K and V blocks are
// gathered page by page with cp.async into two stages of shared memory; Q.K^T and P.V are mma.sync m16n8k16.
// The sink (one more term exp(0) in the denominator) enters a row's running maximum and sum once.
#include "common.cuh"

#if !defined(MRS_HEAD_DIM) || !defined(MRS_VALUE_DIM)
#error "compile with -DMRS_HEAD_DIM=<key head size> -DMRS_VALUE_DIM=<value head size>"
#endif

namespace {

#ifndef MRS_VALUES_IN_KEYS
#define MRS_VALUES_IN_KEYS 0
#endif
constexpr int D = MRS_HEAD_DIM, E = MRS_VALUE_DIM;
constexpr bool IN_KEYS = MRS_VALUES_IN_KEYS != 0;
constexpr int VW = IN_KEYS ? D : E;            // elements of a row of the tile that holds the values
static_assert(D % 16 == 0 && D >= 16 && D <= (IN_KEYS ? 640 : 256) && E % 16 == 0 && E >= 16 && E <= 256 && (!IN_KEYS || E <= D),
              "head sizes: multiples of 16, keys up to 256 (640 with the values inside), values up to 256");
constexpr int THREADS = 128;
constexpr int ROWS_WIDE = 64, ROWS_NARROW = 16;
constexpr int KV_WIDE = 32;            // keys a block in rows mode: small blocks leave room for three or four CTAs an SM
constexpr int KV_NARROW = 64;
constexpr float LOG2E = 1.4426950408889634f;

// Elements between the rows of a [rows][W] tile in shared memory.  Rows of a multiple of 64 elements are swizzled (their
// 16-byte pieces xor-ed with the row); the others get 16 bytes of padding, which spreads eight consecutive rows over
// all banks (rows of 160 or 288 elements would otherwise meet in the same banks four at a time).
template <int W> constexpr int LD = (W % 64 == 0) ? W : W + 8;
template <int W> __device__ __forceinline__ int tile_offset(int row, int col) {      // element offset in a [rows][W] tile
    const int chunk = col >> 3;
    return row * LD<W> + (((W % 64 == 0) ? (chunk ^ (row & 7)) : chunk) << 3) + (col & 7);
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Tile { int seq, first_token, tokens, pad; };

struct Extras {            // what is put around the scores
    const float* bias;     // [bias_rows, nq] by distance, the last row for every larger one; may be null
    const float* gate;     // [tokens, nq], may be null
    int bias_rows;
    float scale, cap;      // cap 0: none
    int window, keep_first, sink;
    const float* sink_logits;   // [nq]: the sink's term is exp(sink_logits[head]); null: exp(0)
    int chunk;                  // > 0 (and no window): a query sees the keys of its own chunk of positions only
};

// The sink's logit of a query head, in units of log 2.
__device__ __forceinline__ float sink_of(const Extras& x, int head) { return x.sink_logits ? x.sink_logits[head] * LOG2E : 0.0f; }

// Keys [key0, key0 + KV) of one kv head into a [KV][W] shared tile; rows at or beyond `key_end` or on a page that was
// given back are zeros.
template <int KV, int W>
__device__ __forceinline__ void load_kv_block(bf16* dst, const bf16* __restrict__ cache, const int* __restrict__ pages, int key0,
                                              int key_end, int kv_head, int nkv, int page_size, int page_shift) {
    constexpr int CHUNKS = W / 8;
    for (int idx = threadIdx.x; idx < KV * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const int key = key0 + row;
        bool valid = key < key_end;
        const bf16* src = cache;
        if (valid) {
            const int page = pages[key >> page_shift];
            valid = page >= 0;
            if (valid) src = cache + (((size_t)page * nkv + kv_head) * page_size + (key & (page_size - 1))) * W + chunk * 8;
        }
        cp_async16(dst + tile_offset<W>(row, chunk * 8), src, valid);
    }
}

template <int ROWS>
__device__ __forceinline__ void load_q_tile(bf16* q_tile, const bf16* __restrict__ q, const Tile& tile, int rows, int group,
                                            int kv_head, int nq) {
    constexpr int CHUNKS = D / 8;
    for (int idx = threadIdx.x; idx < ROWS * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const bool valid = row < rows;
        const bf16* src = q;
        if (valid) src = q + ((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + chunk * 8;
        cp_async16(q_tile + tile_offset<D>(row, chunk * 8), src, valid);
    }
}

template <int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const bf16* q_tile, int q_row0, const bf16* k_tile, int key_row0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, q_tile + tile_offset<D>(q_row0 + (lane & 15), kk * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, k_tile + tile_offset<D>(key_row0 + nt * 8 + (lane & 7) + ((lane >> 4) << 3), kk * 16 + ((lane >> 3) & 1) * 8));
            mma_bf16(s[nt], a, b[0], b[1]);
            mma_bf16(s[nt + 1], a, b[2], b[3]);
        }
    }
}

template <int NT>
__device__ __forceinline__ void pv_product(float (&o)[E / 8][4], const float (&s)[NT][4], const bf16* v_tile, int key_row0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < E / 8; dt += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_tile + tile_offset<VW>(key_row0 + kk * 16 + (lane & 15), dt * 8 + (lane >> 4) * 8));
            mma_bf16(o[dt], a, b[0], b[1]);
            mma_bf16(o[dt + 1], a, b[2], b[3]);
        }
    }
}

// Scales, caps, biases and masks the scores of one warp (in units of log 2 afterwards), updates the running maximum and
// sum of its two rows (lane / 4 and lane / 4 + 8), rescales the accumulator and turns the scores into weights.
template <int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[E / 8][4], float (&row_max)[2], float (&row_sum)[2],
                                             const int (&row_pos)[2], const int (&row_head)[2], const int (&row_lo)[2], int key0,
                                             int key_end, int nq, const Extras& x) {
    const int t = threadIdx.x & 3;
    float block_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + 2 * t + (e & 1);
            const int pos = row_pos[e >> 1];
            const int back = pos - key;
            const bool seen = back >= 0 && key < key_end && key >= row_lo[e >> 1] && (x.window <= 0 || back < x.window || key < x.keep_first);
            float v = -CUDART_INF_F;
            if (seen) {
                v = s[nt][e] * x.scale;
                if (x.cap > 0.0f) v = x.cap * tanhf(v / x.cap);
                if (x.bias) v += x.bias[(size_t)min(back, x.bias_rows - 1) * nq + row_head[e >> 1]];
                v *= LOG2E;
            }
            s[nt][e] = v;
            block_max[e >> 1] = fmaxf(block_max[e >> 1], v);
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 1));
        block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 2));
        const float new_max = fmaxf(row_max[r], block_max[r]);
        const float base = new_max == -CUDART_INF_F ? 0.0f : new_max;
        const float alpha = exp2f(row_max[r] - base);
        row_max[r] = new_max;
        float sum = 0.0f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s[nt][2 * r] = exp2f(s[nt][2 * r] - base);
            s[nt][2 * r + 1] = exp2f(s[nt][2 * r + 1] - base);
            sum += s[nt][2 * r] + s[nt][2 * r + 1];
        }
        row_sum[r] = row_sum[r] * alpha + sum;      // the sum over the quad's lanes is taken at the end
#pragma unroll
        for (int dt = 0; dt < E / 8; ++dt) {
            o[dt][2 * r] *= alpha;
            o[dt][2 * r + 1] *= alpha;
        }
    }
}

// The key blocks of a tile, in units of KV positions: `kept` blocks from 0 on, then blocks [window_first, last).
struct Blocks {
    int kept, window_first, count;
    __device__ __forceinline__ int at(int i) const { return i < kept ? i : window_first + (i - kept); }
};
__device__ __forceinline__ Blocks blocks_of(int first_pos, int key_end, int kv, const Extras& x) {
    Blocks b;
    const int key_begin = x.chunk > 0 ? (first_pos / x.chunk) * x.chunk : (x.window > 0 ? max(0, first_pos - x.window + 1) : 0);
    b.window_first = key_begin / kv;
    const int kept_keys = x.window > 0 ? min(x.keep_first, key_begin) : 0;
    b.kept = min((kept_keys + kv - 1) / kv, b.window_first);
    b.count = b.kept + (key_end + kv - 1) / kv - b.window_first;
    return b;
}

// With the values inside wide key rows (256 of them) a warp's sums alone are 128 registers and the kernel takes 240: two
// CTAs an SM.  Held to 168 registers it spills a few words and runs three CTAs, and is slower (2,048 tokens of 16 heads,
// rows of 288: 255 against 206 us).
__global__ void __launch_bounds__(THREADS) attention_biased_rows_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, const int* __restrict__ positions,
    const int* __restrict__ block_table, int table_width, const Tile* __restrict__ tiles, bf16* __restrict__ out, int nq, int nkv,
    int page_size, int page_shift, Extras x) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);
    bf16* k_tiles = q_tile + ROWS_WIDE * LD<D>;
    bf16* v_tiles = IN_KEYS ? k_tiles : k_tiles + 2 * KV_WIDE * LD<D>;
    constexpr int NT = KV_WIDE / 8;

    const Tile tile = tiles[blockIdx.x];
    if (tile.tokens <= 0) return;
    const int kv_head = blockIdx.y, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)tile.seq * table_width;
    const int rows = tile.tokens * group;
    load_q_tile<ROWS_WIDE>(q_tile, q, tile, rows, group, kv_head, nq);
    const int first_pos = positions[tile.first_token], last_pos = positions[tile.first_token + tile.tokens - 1];
    const int key_end = last_pos + 1;
    const Blocks blocks = blocks_of(first_pos, key_end, KV_WIDE, x);

    int row_pos[2], row_head[2], row_lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        row_pos[r] = row < rows ? positions[tile.first_token + row / group] : last_pos;
        row_head[r] = kv_head * group + row % group;
        row_lo[r] = x.chunk > 0 ? (row_pos[r] / x.chunk) * x.chunk : 0;
    }
    float o[E / 8][4];
#pragma unroll
    for (int dt = 0; dt < E / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
    float row_max[2], row_sum[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_max[r] = x.sink ? sink_of(x, row_head[r]) : -CUDART_INF_F;
        row_sum[r] = x.sink && (lane & 3) == 0 ? 1.0f : 0.0f;
    }

    if (blocks.count > 0) {
        load_kv_block<KV_WIDE, D>(k_tiles, k_cache, pages, blocks.at(0) * KV_WIDE, key_end, kv_head, nkv, page_size, page_shift);
        if constexpr (!IN_KEYS)
            load_kv_block<KV_WIDE, E>(v_tiles, v_cache, pages, blocks.at(0) * KV_WIDE, key_end, kv_head, nkv, page_size, page_shift);
    }
    cp_async_commit();
    for (int i = 0; i < blocks.count; ++i) {
        const int stage = i & 1;
        if (i + 1 < blocks.count) {
            load_kv_block<KV_WIDE, D>(k_tiles + (stage ^ 1) * KV_WIDE * LD<D>, k_cache, pages, blocks.at(i + 1) * KV_WIDE, key_end, kv_head, nkv, page_size, page_shift);
            if constexpr (!IN_KEYS)
                load_kv_block<KV_WIDE, E>(v_tiles + (stage ^ 1) * KV_WIDE * LD<E>, v_cache, pages, blocks.at(i + 1) * KV_WIDE, key_end, kv_head, nkv, page_size, page_shift);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = blocks.at(i) * KV_WIDE;
        const int warp_last_pos = __shfl_sync(0xffffffffu, row_pos[1], 28);
        if (key0 <= warp_last_pos) {
            float s[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
            qk_product<NT>(s, q_tile, warp * 16, k_tiles + stage * KV_WIDE * LD<D>, 0);
            softmax_step<NT>(s, o, row_max, row_sum, row_pos, row_head, row_lo, key0, key_end, nq, x);
            pv_product<NT>(o, s, v_tiles + stage * KV_WIDE * LD<VW>, 0);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        if (row >= rows) continue;
        const int token = tile.first_token + row / group;
        const float factor = (sum > 0.0f ? 1.0f / sum : 0.0f) * (x.gate ? x.gate[(size_t)token * nq + row_head[r]] : 1.0f);
        bf16* dst = out + ((size_t)token * nq + row_head[r]) * E;
#pragma unroll
        for (int dt = 0; dt < E / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[dt][2 * r] * factor, o[dt][2 * r + 1] * factor);
        }
    }
}

__global__ void __launch_bounds__(THREADS) attention_biased_keys_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, const int* __restrict__ positions,
    const int* __restrict__ block_table, int table_width, const Tile* __restrict__ tiles, bf16* __restrict__ out, int nq, int nkv,
    int page_size, int page_shift, Extras x, float* __restrict__ part_o, float* __restrict__ part_ml, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);
    bf16* k_tiles = q_tile + ROWS_NARROW * LD<D>;
    bf16* v_tiles = IN_KEYS ? k_tiles : k_tiles + 2 * KV_NARROW * LD<D>;
    constexpr int NT = 2;

    const Tile tile = tiles[blockIdx.x];
    if (tile.tokens <= 0) return;
    const int kv_head = blockIdx.y, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)tile.seq * table_width;
    const int rows = tile.tokens * group;
    load_q_tile<ROWS_NARROW>(q_tile, q, tile, rows, group, kv_head, nq);
    const int first_pos = positions[tile.first_token], last_pos = positions[tile.first_token + tile.tokens - 1];
    const int key_end = last_pos + 1;
    const Blocks blocks = blocks_of(first_pos, key_end, KV_NARROW, x);
    // with `splits` CTAs a tile the blocks are dealt in runs; the partial results meet in `attention_biased_combine_kernel`
    const int split = blockIdx.z, share = (blocks.count + splits - 1) / splits;
    const int block_first = min(blocks.count, split * share), block_last = min(blocks.count, block_first + share);

    int row_pos[2], row_head[2], row_lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + 8 * r;
        row_pos[r] = row < rows ? positions[tile.first_token + row / group] : last_pos;
        row_head[r] = kv_head * group + row % group;
        row_lo[r] = x.chunk > 0 ? (row_pos[r] / x.chunk) * x.chunk : 0;
    }
    float o[E / 8][4];
#pragma unroll
    for (int dt = 0; dt < E / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
    float row_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, row_sum[2] = {0.0f, 0.0f};

    if (block_first < block_last) {
        load_kv_block<KV_NARROW, D>(k_tiles, k_cache, pages, blocks.at(block_first) * KV_NARROW, key_end, kv_head, nkv, page_size, page_shift);
        if constexpr (!IN_KEYS)
            load_kv_block<KV_NARROW, E>(v_tiles, v_cache, pages, blocks.at(block_first) * KV_NARROW, key_end, kv_head, nkv, page_size, page_shift);
    }
    cp_async_commit();
    for (int i = block_first; i < block_last; ++i) {
        const int stage = (i - block_first) & 1;
        if (i + 1 < block_last) {
            load_kv_block<KV_NARROW, D>(k_tiles + (stage ^ 1) * KV_NARROW * LD<D>, k_cache, pages, blocks.at(i + 1) * KV_NARROW, key_end, kv_head, nkv, page_size, page_shift);
            if constexpr (!IN_KEYS)
                load_kv_block<KV_NARROW, E>(v_tiles + (stage ^ 1) * KV_NARROW * LD<E>, v_cache, pages, blocks.at(i + 1) * KV_NARROW, key_end, kv_head, nkv, page_size, page_shift);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = blocks.at(i) * KV_NARROW + warp * 16;
        if (key0 < key_end) {
            float s[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
            qk_product<NT>(s, q_tile, 0, k_tiles + stage * KV_NARROW * LD<D>, warp * 16);
            softmax_step<NT>(s, o, row_max, row_sum, row_pos, row_head, row_lo, key0, key_end, nq, x);
            pv_product<NT>(o, s, v_tiles + stage * KV_NARROW * LD<VW>, warp * 16);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the four warps through shared memory: [4][16][E] sums and [4][16][2] (maximum, sum); the sink joins here
    float* merge_o = reinterpret_cast<float*>(k_tiles);
    float* merge_ml = merge_o + 4 * ROWS_NARROW * E;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = (lane >> 2) + 8 * r;
        if ((lane & 3) == 0) {
            merge_ml[(warp * ROWS_NARROW + row) * 2] = row_max[r];
            merge_ml[(warp * ROWS_NARROW + row) * 2 + 1] = sum;
        }
#pragma unroll
        for (int dt = 0; dt < E / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            merge_o[(warp * ROWS_NARROW + row) * E + col] = o[dt][2 * r];
            merge_o[(warp * ROWS_NARROW + row) * E + col + 1] = o[dt][2 * r + 1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS_NARROW * E; idx += THREADS) {
        const int row = idx / E, col = idx % E;
        if (row >= rows) continue;
        const bool with_sink = x.sink && splits == 1;          // among several CTAs the sink joins in the combine kernel
        const float sink_logit = with_sink ? sink_of(x, kv_head * group + row % group) : 0.0f;
        float m = with_sink ? sink_logit : -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, merge_ml[(w * ROWS_NARROW + row) * 2]);
        const float base = m == -CUDART_INF_F ? 0.0f : m;
        float sum = with_sink ? exp2f(sink_logit - base) : 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(merge_ml[(w * ROWS_NARROW + row) * 2] - base);
            sum += merge_ml[(w * ROWS_NARROW + row) * 2 + 1] * f;
            acc += merge_o[(w * ROWS_NARROW + row) * E + col] * f;
        }
        if (splits > 1) {
            const size_t slot = (((size_t)blockIdx.x * nkv + kv_head) * splits + split) * ROWS_NARROW + row;
            part_o[slot * E + col] = acc;
            if (col == 0) part_ml[slot * 2] = m, part_ml[slot * 2 + 1] = sum;
            continue;
        }
        const int token = tile.first_token + row / group, head = kv_head * group + row % group;
        const float factor = (sum > 0.0f ? 1.0f / sum : 0.0f) * (x.gate ? x.gate[(size_t)token * nq + head] : 1.0f);
        out[((size_t)token * nq + head) * E + col] = __float2bfloat16_rn(acc * factor);
    }
}

// Merges the partial results of a tile's `splits` CTAs, adds the sink and applies the gate.
__global__ void __launch_bounds__(THREADS) attention_biased_combine_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const Tile* __restrict__ tiles, bf16* __restrict__ out,
    const float* __restrict__ gate, int nq, int nkv, int splits, int sink, const float* __restrict__ sink_logits) {
    pdl_launch_dependents();
    pdl_wait();
    const Tile tile = tiles[blockIdx.x];
    const int kv_head = blockIdx.y, group = nq / nkv, rows = tile.tokens * group;
    const size_t base_slot = ((size_t)blockIdx.x * nkv + kv_head) * splits * ROWS_NARROW;
    const int row = blockIdx.z;                       // a CTA a row: few tiles still fill the GPU
    if (row >= rows) return;
    const float sink_logit = sink && sink_logits ? sink_logits[kv_head * group + row % group] * LOG2E : 0.0f;
    for (int col = threadIdx.x; col < E; col += THREADS) {
        float m = sink ? sink_logit : -CUDART_INF_F;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base_slot + (size_t)s * ROWS_NARROW + row) * 2]);
        const float base = m == -CUDART_INF_F ? 0.0f : m;
        float sum = sink ? exp2f(sink_logit - base) : 0.0f, acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const size_t slot = base_slot + (size_t)s * ROWS_NARROW + row;
            const float f = exp2f(part_ml[slot * 2] - base);
            sum += part_ml[slot * 2 + 1] * f;
            acc += part_o[slot * E + col] * f;
        }
        const int token = tile.first_token + row / group, head = kv_head * group + row % group;
        const float factor = (sum > 0.0f ? 1.0f / sum : 0.0f) * (gate ? gate[(size_t)token * nq + head] : 1.0f);
        out[((size_t)token * nq + head) * E + col] = __float2bfloat16_rn(acc * factor);
    }
}

constexpr int KV_ROW = LD<D> + (IN_KEYS ? 0 : LD<E>);      // elements of shared memory a key
constexpr size_t smem_rows = (size_t)(ROWS_WIDE * LD<D> + 2 * KV_WIDE * KV_ROW) * sizeof(bf16);
constexpr size_t smem_keys_tiles = (size_t)(ROWS_NARROW * LD<D> + 2 * KV_NARROW * KV_ROW) * sizeof(bf16);
constexpr size_t smem_keys_merge = (size_t)ROWS_NARROW * LD<D> * sizeof(bf16) + (size_t)(4 * ROWS_NARROW * E + 4 * ROWS_NARROW * 2) * sizeof(float);
constexpr size_t smem_keys = smem_keys_tiles > smem_keys_merge ? smem_keys_tiles : smem_keys_merge;

int page_shift_of(int page_size) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    return (1 << shift) == page_size ? shift : -1;
}

}  // namespace

MRS_EXPORT int mrs_attention_biased_mma_key_dim() { return D; }
MRS_EXPORT int mrs_attention_biased_mma_value_dim() { return E; }
MRS_EXPORT int mrs_attention_biased_mma_values_in_keys() { return IN_KEYS ? 1 : 0; }

// narrow != 0: tiles of up to 16 / group tokens (keys mode); else tiles of up to 64 / group tokens (rows mode).
// Scratch floats of `splits` > 1 CTAs a tile (tiles of 16 rows only).
MRS_EXPORT long long mrs_attention_biased_mma_scratch_floats(int tiles, int nkv, int splits) {
    return splits <= 1 ? 0 : (long long)tiles * nkv * splits * ROWS_NARROW * (E + 2);
}

MRS_EXPORT int mrs_attention_biased_mma(int narrow, const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                        const int* block_table, int table_width, const int* tiles, int num_tiles, void* out,
                                        const float* bias, int bias_rows, const float* gate, int nq, int nkv, int page_size,
                                        float scale, float cap, int window, int keep_first, int sink, int splits, float* scratch,
                                        const float* sink_logits, int chunk, void* stream) {
    if (num_tiles <= 0) return 0;
    if (splits < 1 || splits > 65535 || (splits > 1 && (!narrow || !scratch)) || (!IN_KEYS && !v_cache)) return MRS_BAD_ARGUMENT;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || nkv <= 0 || nq % nkv || nq / nkv > (narrow ? ROWS_NARROW : ROWS_WIDE) || (bias && bias_rows <= 0) || window < 0 ||
        keep_first < 0 || chunk < 0 || (chunk > 0 && window > 0) || (sink_logits && !sink))
        return MRS_BAD_ARGUMENT;
    Extras x;
    x.bias = bias, x.gate = gate, x.bias_rows = bias_rows, x.scale = scale, x.cap = cap, x.window = window, x.keep_first = keep_first;
    x.sink = sink, x.sink_logits = sink_logits, x.chunk = chunk;
    static bool configured[2] = {false, false};
    if (!configured[narrow ? 1 : 0]) {
        cudaError_t e = narrow
            ? cudaFuncSetAttribute(attention_biased_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_keys)
            : cudaFuncSetAttribute(attention_biased_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows);
        if (e != cudaSuccess) return (int)e;
        configured[narrow ? 1 : 0] = true;
    }
    if (narrow) {
        float* part_o = scratch;
        float* part_ml = scratch ? scratch + (size_t)num_tiles * nkv * splits * ROWS_NARROW * E : nullptr;
        MRS_LAUNCH(attention_biased_keys_kernel, dim3(num_tiles, nkv, splits), THREADS, smem_keys, stream, (const bf16*)q,
                   (const bf16*)k_cache, (const bf16*)v_cache, positions, block_table, table_width, (const Tile*)tiles, (bf16*)out, nq, nkv,
                   page_size, shift, x, part_o, part_ml, splits);
        if (splits > 1)
            MRS_LAUNCH(attention_biased_combine_kernel, dim3(num_tiles, nkv, ROWS_NARROW), E < THREADS ? 32 * ((E + 31) / 32) : THREADS, 0, stream, (const float*)part_o,
                       (const float*)part_ml, (const Tile*)tiles, (bf16*)out, gate, nq, nkv, splits, sink, sink_logits);
    } else
        MRS_LAUNCH(attention_biased_rows_kernel, dim3(num_tiles, nkv), THREADS, smem_rows, stream, (const bf16*)q, (const bf16*)k_cache,
                   (const bf16*)v_cache, positions, block_table, table_width, (const Tile*)tiles, (bf16*)out, nq, nkv, page_size, shift, x);
    MRS_RETURN_LAUNCH_STATUS();
}
